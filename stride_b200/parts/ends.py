"""The two ends of a decoder: the token embedding and the output head.

Embedding: h = widen(table[token]), no scaling (arhaamatiq/stride src/kernels.cu:98-116).
Head: logits = W x for the rows that want logits; W is `lm_head.weight` if the
checkpoint has it, else the embedding table (src/model.cpp:228-232).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import Part, register_part
from .spec import TensorPlan


@register_part("embedding", "lookup")
class Embedding(Part):
    """params: vocab_size, hidden_size. tensors: weight."""
    graph_safe = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight = None

    def tensor_plan(self):
        return {self.spec.tensors["weight"]: TensorPlan((self.vocab, self.hidden))}

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def weight_bytes(self):
        return 0   # a step reads one row per token, not the table

    def forward(self, ctx, out):
        ops.embed(ctx.token_ids, self.weight, out, ctx.slots if ctx.sampled is not None else None, ctx.sampled)

    def emit(self, program, out, sampled):
        program.add("elementwise", "sb_op_embed", [self.weight, self.weight.dtype, out, self.hidden, self.weight.shape[0], sampled])


@register_part("head", "linear")
class LinearHead(Part):
    """params: vocab_size, hidden_size, tied (True: always the embedding table; False: its own
    matrix is required; None: its own matrix if the checkpoint has one). tensors: weight, tied_to."""
    graph_safe = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = spec.params.get("tied")
        self.linear = None

    def tensor_plan(self):
        t = self.spec.tensors
        plan = {t["tied_to"]: TensorPlan((self.vocab, self.hidden))} if self.tied is not False else {}
        if self.tied is not True:
            plan[t["weight"]] = TensorPlan((self.vocab, self.hidden), optional=self.tied is None)
        return plan

    def bind(self, tensors):
        t = self.spec.tensors
        own = tensors.get(t["weight"]) if self.tied is not True else None
        self.is_tied = own is None
        self.linear = Linear(own if own is not None else tensors[t["tied_to"]], self.env.compute_dtype)

    def weight_bytes(self):
        return self.linear.weight_bytes()

    def forward(self, x, logits):
        """logits[count, vocab] float32 = x . W^T for the normed rows x."""
        self.linear.forward(x, logits)

    def emit(self, program, x, logits):
        self.linear.emit(program, x, logits, wanted_rows=True)
