"""Arrangements of a layer's parts around the residual stream.

`pre_norm` is GPT-2's: `x -> norm1 -> mixer -> +x -> norm2 -> feed-forward -> +x`, the residual
sums in float32 (graph_ir.cpp:732-756, the sequential branch; operand order x then the
branch's output, :754-756).  The mixer and the feed-forward add into the stream themselves so that
their last projection can do the sum in its epilogue.
"""
from __future__ import annotations

from .base import Block, register_part


class PreNormBlock(Block):
    def __init__(self, norm1, mixer, norm2, ffn, **more_norms):
        if norm1 is None or norm2 is None or more_norms:
            raise ValueError("block 'pre_norm' has exactly two norms: one before the mixer, one before the feed-forward")
        super().__init__(norm1, mixer, norm2, ffn)


    def forward(self, ctx, x, app):
        announce = getattr(ctx.ops, "announce_weights", None)
        if announce is not None:    # a hint: this block's matrices in the order they are streamed, then what follows
            announce(self.mixer.stream_weights() + self.ffn.stream_weights() + list(getattr(ctx, "next_weights", ())))
        h = self.norm1.forward(ctx, x, ctx.dtype)
        x = self.mixer.forward(ctx, h, x, app)
        h = self.norm2.forward(ctx, x, ctx.dtype)
        return self.ffn.forward(ctx, h, x)


register_part("block", "pre_norm", PreNormBlock)
