"""Block arrangements. "prenorm": h += mixer(norm(h)); h += feed_forward(norm(h))
(arhaamatiq/stride src/engine.cpp:166-237)."""
from __future__ import annotations

from .base import Block, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def forward(self, ctx, stream, cache):
        width = stream.h.shape[1]
        x = ctx.workspace.get("block.x", ctx.n, (width,), ctx.act_dtype)
        self.mixer_norm.forward(ctx, stream, x)
        self.mixer.forward(ctx, x, stream, cache)
        self.feed_forward_norm.forward(ctx, stream, x)
        self.feed_forward.forward(ctx, x, stream)

    def emit(self, program, cache):
        ws = program.workspace
        x = ws.get("block.x", ws.max_tokens, (program.h.shape[1],), self.env.act_dtype)
        self.mixer_norm.emit(program, x)
        self.mixer.emit(program, x, cache)
        self.feed_forward_norm.emit(program, x)
        self.feed_forward.emit(program, x)
