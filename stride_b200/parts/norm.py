"""RMSNorm: y = w * (x / sqrt(mean(x^2) + eps)), all in 32-bit
(arhaamatiq/stride src/kernels.cu:119-200: the weight is a plain gain, eps sits inside the root)."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, register_part
from .spec import TensorPlan


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: size, eps. tensors: weight."""
    graph_safe = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def tensor_plan(self):
        return {self.spec.tensors["weight"]: TensorPlan((self.size,))}

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx, stream, out):
        ops.rmsnorm(stream.h, self.weight, self.eps, out, partials=stream.take_pending())

    def kernel_libraries(self):
        return {"norm"}

    def forward_rows(self, rows, out):
        """Norm of a plain [n, size] float32 tensor (the rows gathered for the head)."""
        ops.rmsnorm(rows, self.weight, self.eps, out)

    def _op(self, program, h, pending, out, wanted_rows: bool):
        flat, S, _ = pending if pending is not None else (None, 1, 0)
        phase = None if wanted_rows else (lambda chain: chain.norm(h, pending, self.weight, out, self.size, self.eps))
        program.add("norm", "sb_op_rmsnorm", [h, flat, S, program.few_tokens, self.weight, self.weight.dtype, out, out.dtype, self.size,
                                              int(wanted_rows)], [self.eps], chain=phase)

    def emit(self, program, out):
        self._op(program, program.h, program.take_pending(), out, False)

    def emit_rows(self, program, rows, out):
        self._op(program, rows, None, out, True)
