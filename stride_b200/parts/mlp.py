"""The gated feed-forward of Llama: h += W2 (silu(W1 x) * (W3 x)), silu(a) = a / (1 + exp(-a))
(arhaamatiq/stride src/kernels.cu:329-363, src/numerics.h:33; down projection added to the
residual: src/kernels.cu:294-325). gate_proj = W1, up_proj = W3, down_proj = W2."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import FeedForward, register_part
from .spec import TensorPlan


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, intermediate_size. tensors: gate, up, down."""
    graph_safe = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        self.intermediate = int(spec.params["intermediate_size"])
        self.gate_up = self.down = None

    def tensor_plan(self):
        t = self.spec.tensors
        return {t["gate"]: TensorPlan((self.intermediate, self.hidden)),
                t["up"]: TensorPlan((self.intermediate, self.hidden)),
                t["down"]: TensorPlan((self.hidden, self.intermediate))}

    def bind(self, tensors):
        t = self.spec.tensors
        gate, up = tensors[t["gate"]], tensors[t["up"]]
        if gate.dtype != up.dtype:
            gate, up = gate.to(torch.float32), up.to(torch.float32)
        self.gate_up = Linear(torch.cat([gate, up], dim=0), self.env.compute_dtype)
        self.down = Linear(tensors[t["down"]], self.env.compute_dtype)

    def weight_bytes(self):
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    def kernel_libraries(self):
        return {"gemm_tc"} if self.env.compute_dtype == torch.bfloat16 else {"gemm_f32", "elementwise"}

    def forward(self, ctx, x, stream):
        n, ws = ctx.n, ctx.workspace
        z = ws.get("mlp.z", n, (self.intermediate,), ctx.act_dtype)
        self.gate_up.forward_swiglu(x, z, lambda: ws.get("mlp.gate_up", n, (2 * self.intermediate,), torch.float32))
        self.down.forward_add(z, stream, ws.raw("mlp.down_partials", (self.down.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x):
        ws = program.workspace
        z = ws.get("mlp.z", ws.max_tokens, (self.intermediate,), self.env.act_dtype)
        self.gate_up.emit_swiglu(program, x, z, lambda: ws.get("mlp.gate_up", ws.max_tokens, (2 * self.intermediate,), torch.float32))
        self.down.emit_add(program, z, ws.raw("mlp.down_partials", (self.down.partial_elems(ws.max_tokens),), torch.float32))
