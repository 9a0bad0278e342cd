"""A decoder put together from a `ModelSpec`: embedding, layers run in the order the
schedule gives, final norm and head on the rows whose logits are wanted."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import BuildEnv, part_class
from .context import ResidualStream
from .spec import ModelSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        self.spec, self.env = spec, env
        self.embedding = part_class("embedding", spec.embedding.kind)(spec.embedding, env)
        self.blocks = []
        for i, layer in enumerate(spec.layers):
            block_class = part_class("block", layer.block)
            unknown = [r for r in layer.parts if r not in block_class.ROLES]
            if unknown:
                raise ValueError(f"layer {i}: a '{layer.block}' block has no role {', '.join(unknown)} (its roles: {', '.join(block_class.ROLES)})")
            parts = {role: part_class(block_class.ROLES[role], ps.kind)(ps, env) for role, ps in layer.parts.items()}
            self.blocks.append(block_class(layer, env, parts))
        self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm, env)
        self.head = part_class("head", spec.head.kind)(spec.head, env)
        for i, e in enumerate(spec.schedule):
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, but the model has {len(self.blocks)} layers")
            if e.cache_of is not None and not 0 <= e.cache_of < i:
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")

    @property
    def graph_safe(self) -> bool:
        return (self.embedding.graph_safe and self.final_norm.graph_safe and self.head.graph_safe
                and all(b.all_graph_safe for b in self.blocks))

    def _parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def tensor_plan(self) -> dict:
        plan = {}
        for p in self._parts():
            for name, want in p.tensor_plan().items():
                if name in plan and plan[name].shape != want.shape:
                    raise ValueError(f"tensor '{name}' is expected with shapes {plan[name].shape} and {want.shape}")
                if name not in plan or plan[name].optional:
                    plan[name] = want
        return plan

    def bind(self, tensors: dict) -> None:
        for p in self._parts():
            p.bind(tensors)

    def cache_needs(self) -> list:
        """Per schedule entry: a CacheNeed, None, or ("shared", j)."""
        needs = []
        for e in self.spec.schedule:
            needs.append(("shared", e.cache_of) if e.cache_of is not None else self.blocks[e.layer].cache_need())
        return needs

    def kernel_libraries(self) -> set:
        names = {"elementwise", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}
        for p in self._parts():
            names |= p.kernel_libraries()
        if self.env.decode_chain and {"gemm_tc", "attention_tc"} <= names:
            names.add("decode_chain")
        return names

    def weight_bytes(self) -> int:
        """Bytes of weights that one decode step reads: every scheduled layer once, the final
        norm and the head (arhaamatiq/stride counts the same, src/model.cpp:198,235)."""
        total = self.final_norm.weight_bytes() + self.head.weight_bytes()
        for e in self.spec.schedule:
            total += self.blocks[e.layer].weight_bytes()
        return total

    def forward(self, ctx, caches: list, logit_rows: torch.Tensor, count: int):
        """Run the step's tokens through the model; returns logits [count, vocab] float32 for the
        rows listed in `logit_rows` (int32, device), or None when count is 0."""
        ws, H = ctx.workspace, self.spec.hidden_size
        stream = ResidualStream(ws.get("model.h", ctx.n, (H,), torch.float32))
        self.embedding.forward(ctx, stream.h)
        for i, e in enumerate(self.spec.schedule):
            self.blocks[e.layer].forward(ctx, stream, caches[i])
        if count == 0:
            return None        # pending partial sums die with the stream: nobody reads h after the last layer
        rows = ws.raw("model.head_rows", (ws.max_tokens, H), torch.float32)[:count]
        ops.gather_rows(stream.h, logit_rows, rows, partials=stream.take_pending())
        x = ws.raw("model.head_x", (ws.max_tokens, H), ctx.act_dtype)[:count]
        self.final_norm.forward_rows(rows, x)
        if count > self.env.max_logit_rows:
            raise ValueError(f"logits are wanted at {count} places, more than the engine's max_logit_rows {self.env.max_logit_rows}")
        logits = ws.raw("model.logits", (self.env.max_logit_rows, self.spec.vocab_size), torch.float32)[:count]
        self.head.forward(x, logits)
        return logits

    def emit(self, program, caches: list, sampled) -> torch.Tensor:
        """The whole step as operations of the native step program (what `forward` launches, in the same order);
        returns the buffer [max_logit_rows, vocab] the logits of the wanted rows land in. Raises `NotNative` when a part
        has no native form."""
        ws, H = program.workspace, self.spec.hidden_size
        program.h = ws.get("model.h", ws.max_tokens, (H,), torch.float32)
        self.embedding.emit(program, program.h, sampled)
        chained = self.env.decode_chain and "decode_chain" in self.kernel_libraries()
        if chained:
            # every operation of the layers also names its phase of the decode chain; if all of them have one, one
            # kernel stands for the layers in steps of decoded tokens only
            program.begin_chain()
        for i, e in enumerate(self.spec.schedule):
            self.blocks[e.layer].emit(program, caches[i])
        if chained:
            program.end_chain()
        rows = ws.raw("model.head_rows", (ws.max_tokens, H), torch.float32)
        flat, S, _ = program.take_pending() or (None, 1, 0)
        program.add("elementwise", "sb_op_gather_rows", [program.h, flat, S, program.few_tokens, rows, H])
        x = ws.raw("model.head_x", (ws.max_tokens, H), self.env.act_dtype)
        self.final_norm.emit_rows(program, rows, x)
        logits = ws.raw("model.logits", (self.env.max_logit_rows, self.spec.vocab_size), torch.float32)
        self.head.emit(program, x, logits)
        return logits
