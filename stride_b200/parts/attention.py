"""Grouped-query attention over the paged cache.

One step of it, for all tokens of the batch at once: q, k, v = W x; rotate q and k
by the position encoding; append k and v to the request's pages; every token then
attends to the keys of its own request at positions first..pos (its own included),
first = 0 or pos - window + 1; the result goes through the output projection
into the residual. Order and formulas as in arhaamatiq/stride (Qkv: src/kernels.cu:204-284;
attention: src/kernel_common.h:90-309; scale = float(pow(double(D), -0.5)), src/engine.cpp:151;
output projection added to the residual: src/kernels.cu:294-325). The token's own key is in the
cache before attention runs, so a portion of a prompt needs no mask tensor.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import ops
from ..kernels.linear import Linear
from ..kernels.native import NO_PHASE
from .base import CacheNeed, Mixer, part_class, register_part
from .spec import TensorPlan


@register_part("mixer", "attention")
class AttentionMixer(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (0 = all keys),
    position (a PartSpec of category "position", or None), scale (default head_dim ** -0.5).
    tensors: q, k, v, o."""
    graph_safe = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = int(p.get("window", 0) or 0)
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"attention: {self.num_heads} heads do not divide into {self.num_kv_heads} key/value heads")
        scale = p.get("scale")
        self.scale = float(np.float32(math.pow(float(self.head_dim), -0.5))) if scale is None else float(scale)
        pos = p.get("position")
        self.position = part_class("position", pos.kind)(pos, env) if pos is not None else None
        self.qkv = self.o = None

    @property
    def qkv_width(self):
        return (self.num_heads + 2 * self.num_kv_heads) * self.head_dim

    def tensor_plan(self):
        t, D = self.spec.tensors, self.head_dim
        plan = {t["q"]: TensorPlan((self.num_heads * D, self.hidden)),
                t["k"]: TensorPlan((self.num_kv_heads * D, self.hidden)),
                t["v"]: TensorPlan((self.num_kv_heads * D, self.hidden)),
                t["o"]: TensorPlan((self.hidden, self.num_heads * D))}
        if self.position is not None:
            plan.update(self.position.tensor_plan())      # a position part may have tensors of its own (a learned table)
        return plan

    def bind(self, tensors):
        t = self.spec.tensors
        q, k, v = tensors[t["q"]], tensors[t["k"]], tensors[t["v"]]
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = (w.to(torch.float32) for w in (q, k, v))
        self.qkv = Linear(torch.cat([q, k, v], dim=0), self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        if self.position is None:
            # No rotation: a table of cos = 1, sin = 0 is never read because rotary_dim is 0.
            self._cos_sin, self._rotary = torch.zeros(1, device=self.env.device), 0
        else:
            self.position.bind(tensors)
            table, rotary = getattr(self.position, "cos_sin", None), getattr(self.position, "rotary_dim", None)
            if not isinstance(table, torch.Tensor) or rotary is None or table.dim() != 3 or table.shape[-1] != 2 \
                    or rotary % 2 or not 0 <= rotary <= self.head_dim or (rotary and table.shape[1] != rotary // 2):
                raise TypeError(f"the position part '{self.spec.params['position'].kind}' does not offer what the attention mixer's kernels "
                                f"read: cos_sin [positions, rotary_dim / 2, 2] float32 and an even rotary_dim <= head_dim {self.head_dim} "
                                f"(see parts.base.PositionEncoding); an encoding of another nature needs a mixer of its own")
            self._cos_sin, self._rotary = table, int(rotary)

    def weight_bytes(self):
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    def cache_need(self):
        return CacheNeed("pages", kv_heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window,
                         dtype=self.env.act_dtype)

    @staticmethod
    def _tc_plan(ctx, G: int, tile_rows: int = 64):
        """(work list on the device, tiles, items, chunks) of the tensor-core attention kernels for this
        step: entries of at most 16 // G tokens go to the decode kernel (one item each), longer ones are
        cut into tiles of tile_rows // G positions. Made once per step and shared by all layers of this ratio."""
        key = ("attention_tc_plan", G, tile_rows)
        plan = ctx.shared.get(key)
        if plan is None and ctx.static_keys:
            E = len(ctx.entry_length)
            plan = (ctx.workspace.iota(E), 0, E, (ctx.static_keys + 255) // 256)
            ctx.shared[key] = plan
        if plan is None:
            ppt, short = tile_rows // G, 16 // G
            tiled, items, last = [], [], 0
            for e, (L, p0) in enumerate(zip(ctx.entry_length, ctx.entry_first_pos)):
                if L <= short:
                    items.append(e)
                    last = max(last, p0 + L - 1)
                else:
                    tiled += [(p0 + min(L, (t + 1) * ppt), e, t) for t in range((L + ppt - 1) // ppt)]
            # the tiles that see the most keys first: CTAs start in this order, and the short ones fill the end
            tiled.sort(key=lambda k: -k[0])
            tiles = [x for _, e, t in tiled for x in (e, t)]
            work = ctx.upload_ints(np.asarray(tiles + items, dtype=np.int32))
            plan = (work, len(tiles) // 2, len(items), last // 256 + 1 if items else 0)
            ctx.shared[key] = plan
        return plan

    def kernel_libraries(self):
        if self.env.compute_dtype != torch.bfloat16:
            return {"gemm_f32", "elementwise", "attention_generic"}
        G = self.num_heads // self.num_kv_heads
        if self.head_dim in (64, 128) and G <= 16:
            return {"gemm_tc", "elementwise", "attention_tc", "attention_tc5"}
        return {"gemm_tc", "elementwise", "attention_generic"}

    def forward(self, ctx, x, stream, cache):
        n, ws, D = ctx.n, ctx.workspace, self.head_dim
        qkv = self.qkv.forward_partials(x, ws.raw("attn.qkv", (self.qkv.partial_elems(ws.max_tokens),), torch.float32))
        mixed = ws.get("attn.out", n, (self.num_heads * D,), ctx.act_dtype)
        G = self.num_heads // self.num_kv_heads
        tensor_core = ctx.act_dtype == torch.bfloat16 and D in (64, 128) and G <= 16
        plan = None
        if tensor_core:
            tc5 = ops.attention_tc5_supported(self.num_heads, self.num_kv_heads, D, cache.page_size)
            plan = self._tc_plan(ctx, G, 128 if tc5 else 64)
        if (plan is not None and plan[1] == 0 and cache.writes and self._rotary == D
                and plan[2] * self.num_kv_heads * plan[3] <= ops.attention_decode_rope_limit()):
            # only decoded tokens and very short portions, few enough for all CTAs to run at once: rotation and append
            # happen inside the decode kernel (the same bits; with more CTAs than that the separate kernel is faster)
            work, _, n_items, chunks = plan
            scratch = ws.grow("attn.scratch", ops.attention_tc_scratch(n_items, self.num_kv_heads, chunks, D), torch.float32)
            counters = ws.raw("attn.counters", (ws.max_tokens * self.num_kv_heads,), torch.int32)
            ops.attention_decode_rope(qkv, self._cos_sin, mixed, cache.pages, cache.block_table, ctx.entry_meta, work, n_items,
                                      chunks, scratch, counters, self.num_heads, self.num_kv_heads, D, self.window, self.scale)
            self.o.forward_add(mixed, stream, ws.raw("attn.o_partials", (self.o.partial_elems(ws.max_tokens),), torch.float32))
            return
        q = ws.get("attn.q", n, (self.num_heads * D,), ctx.act_dtype)
        ops.rope_append(qkv, ctx.positions, ctx.slots, self._cos_sin, self._rotary, q, cache.pages, cache.block_table,
                        self.num_heads, self.num_kv_heads, D, write_kv=cache.writes)
        if tensor_core:
            # prompt portions: the tcgen05 kernel where the page size allows it (tiles of 128 rows), else mma.sync (64 rows);
            # decoded tokens and very short portions: the split-key decode kernel
            work, n_tiles, n_items, chunks = plan
            if tc5 and n_tiles:
                ops.attention_tc5(q, mixed, cache.pages, cache.block_table, ctx.entry_meta, work, n_tiles, self.num_heads,
                                  self.num_kv_heads, D, self.window, self.scale)
                work, n_tiles = work[2 * n_tiles:], 0
            if n_tiles or n_items:
                scratch = ws.grow("attn.scratch", ops.attention_tc_scratch(n_items, self.num_kv_heads, chunks, D), torch.float32)
                counters = ws.raw("attn.counters", (ws.max_tokens * self.num_kv_heads,), torch.int32)
                ops.attention_tc(q, mixed, cache.pages, cache.block_table, ctx.entry_meta, work, n_tiles, n_items, chunks,
                                 scratch, self.num_heads, self.num_kv_heads, D, self.window, self.scale, counters=counters)
        else:
            ops.attention_generic(q, mixed, cache.pages, cache.block_table, ctx.positions, ctx.slots,
                                  self.num_heads, self.num_kv_heads, D, self.window, self.scale)
        self.o.forward_add(mixed, stream, ws.raw("attn.o_partials", (self.o.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x, cache):
        """`forward` as operations of the native step program: the projection, then rotation and append, the
        attention kernels that this shape takes (each finds its share of the step in the step's tile plan, or skips),
        the output projection."""
        ws, env, D = program.workspace, self.env, self.head_dim
        act, T = env.act_dtype, ws.max_tokens
        qkv = ws.raw("attn.qkv", (self.qkv.partial_elems(T),), torch.float32)
        S = self.qkv.emit_partials(program, x, qkv)
        mixed = ws.get("attn.out", T, (self.num_heads * D,), act)
        q = ws.get("attn.q", T, (self.num_heads * D,), act)
        G = self.num_heads // self.num_kv_heads
        tensor_core = act == torch.bfloat16 and D in (64, 128) and G <= 16
        pages, table = cache.pages, cache.block_table
        where = [pages, table, table.shape[1], pages.shape[3], pages.stride(0), pages.stride(1), pages.stride(2)]
        plan = -1
        if tensor_core:
            tc5 = ops.attention_tc5_supported(self.num_heads, self.num_kv_heads, D, cache.page_size)
            fused = cache.writes and self._rotary == D
            plan = program.plan(G, 128 if tc5 else 64, self.num_kv_heads, ops.attention_decode_rope_limit() if fused else -1)
        # (in a step of decoded tokens only, rotation and append can happen inside the attention kernel: the decode chain
        # counts on it, so it takes this mixer only with a fully rotated head and a cache of its own)
        program.add("elementwise", "sb_op_rope_append",
                    [qkv, self.qkv_width, S, program.few_tokens, self._cos_sin, self._rotary, q, q.dtype, pages, pages.dtype, table,
                     table.shape[1], pages.shape[3], pages.stride(0), pages.stride(1), pages.stride(2), self.num_heads,
                     self.num_kv_heads, D, int(cache.writes), plan], chain=NO_PHASE if tensor_core and fused else None)
        if tensor_core:
            if tc5:
                program.add("attention_tc5", "sb_op_attention_tc5",
                            [q, mixed, pages, pages.shape[0], *where[1:], self.num_heads, self.num_kv_heads, D, self.window, plan], [self.scale],
                            chain=NO_PHASE)
            # the decode kernel's chunk records: as many as the step's decode entries and their longest context need
            kv, need = self.num_kv_heads, ops.attention_tc_scratch
            scratch = program.growing_buffer("attn.scratch", torch.float32, (plan, kv, D),
                                             lambda step, k=plan: need(step.plan[k].items, kv, step.plan[k].chunks, D))
            counters = ws.raw("attn.counters", (T * self.num_kv_heads,), torch.int32)
            program.add("attention_tc", "sb_op_attention_tc",
                        [q, mixed, *where, scratch, 0, counters, self.num_heads, self.num_kv_heads, D, self.window, plan,
                         int(tc5), qkv, self.qkv_width, S, program.few_tokens, self._cos_sin], [self.scale],
                        chain=lambda chain: chain.attention(qkv, S, self._cos_sin, mixed, pages, table, scratch, counters, self.num_heads,
                                                            self.num_kv_heads, D, self.window, self.scale, plan))
        else:
            program.add("attention_generic", "sb_op_attention_generic",
                        [q, mixed, q.dtype, *where, self.num_heads, self.num_kv_heads, D, self.window], [self.scale])
        self.o.emit_add(program, mixed, ws.raw("attn.o_partials", (self.o.partial_elems(T),), torch.float32))
