"""Arrangements of a layer's parts around the residual stream.

`pre_norm` is GPT-2's: `x -> norm1 -> mixer -> +x -> norm2 -> feed-forward -> +x`, the residual
sums in float32 (graph_ir.cpp:732-756, the sequential branch; operand order x then the
branch's output, :754-756).  The mixer and the feed-forward add into the stream themselves so that
their last projection can do the sum in its epilogue.
"""
from __future__ import annotations

from .base import Block, register_part


class PreNormBlock(Block):
    ops_only = True

    def forward(self, ctx, x, app):
        h = self.norm1.forward(ctx, x, ctx.dtype, lazy=self.mixer.takes_lazy_norm)
        x = self.mixer.forward(ctx, h, x, app)
        h = self.norm2.forward(ctx, x, ctx.dtype, lazy=self.ffn.takes_lazy_norm)
        return self.ffn.forward(ctx, h, x)


register_part("block", "pre_norm", PreNormBlock)
