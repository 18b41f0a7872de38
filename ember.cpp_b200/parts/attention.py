"""Causal multi-head attention over the cache, with a fused q|k|v projection.

ember.cpp's GPT-2 block: `qkv = h W^T + b`, split into q | k | v by columns
(sizes [H*hd, KV*hd, KV*hd], graph_ir.cpp:733-735), write k and v at their positions, then for
each query the scaled scores over the keys up to its own position, softmax, weighted sum of the
values (graph_ir.cpp:2539-2620; cpu_attention.cpp:92-211), and the output projection whose result
is added to the residual stream (graph_ir.cpp:742, 754).  Query head h reads key/value head
h // (H / KV) (cpu_attention.cpp:127).  With `window` > 0 a query at position p sees positions
p-window+1 .. p (cpu_attention.cpp, swa_visible_ranges).  The scale is a parameter: the
architecture computes it (GPT-2: 1/sqrt(hd), optionally divided by layer+1).
"""
from __future__ import annotations

from .base import CacheNeed, Mixer, WeightSpec, register_part


class CausalAttention(Mixer):

    def __init__(self, prefix: str, width: int, n_heads: int, kv_heads: int, head_dim: int, scale: float,
                 window: int = 0, qkv: str = "c_attn", out: str = "c_proj", stored: str = "in_out",
                 bias: bool = True, init_std: float = 0.02, out_init_std: float = 0.02, bias_init_std: float = 0.01):
        super().__init__(prefix)
        if n_heads % kv_heads:
            raise ValueError(f"attention {prefix!r}: {n_heads} heads are not a multiple of {kv_heads} key/value heads")
        if not 1 <= head_dim <= 256:
            raise ValueError(f"attention {prefix!r}: head size {head_dim} is not in [1, 256]")
        if stored not in ("in_out", "out_in"):
            raise ValueError(f"attention {prefix!r}: stored = {stored!r}")
        self.width, self.n_heads, self.kv_heads, self.head_dim = int(width), int(n_heads), int(kv_heads), int(head_dim)
        self.scale, self.window = float(scale), int(window)
        self.qkv_name, self.out_name, self.stored, self.bias = prefix + qkv, prefix + out, stored, bias
        self.init_std, self.out_init_std, self.bias_init_std = init_std, out_init_std, bias_init_std
        self.q_width = self.n_heads * self.head_dim
        self.qkv_width = (self.n_heads + 2 * self.kv_heads) * self.head_dim
        self.w_qkv = self.b_qkv = self.w_out = self.b_out = None

    def _shape(self, n_in, n_out):
        return (n_in, n_out) if self.stored == "in_out" else (n_out, n_in)

    def weight_specs(self):
        specs = [WeightSpec(self.qkv_name + ".weight", self._shape(self.width, self.qkv_width), std=self.init_std),
                 WeightSpec(self.out_name + ".weight", self._shape(self.q_width, self.width), std=self.out_init_std)]
        if self.bias:
            specs += [WeightSpec(self.qkv_name + ".bias", (self.qkv_width,), std=self.bias_init_std),
                      WeightSpec(self.out_name + ".bias", (self.width,), std=self.bias_init_std)]
        return specs

    def load(self, get, runtime):
        import torch
        if runtime.dtype == torch.bfloat16 and (self.head_dim % 16 or self.width % 8):
            # (the true 32-bit path takes every head size up to 256 and every width)
            raise ValueError(f"attention {self.prefix!r}: the bfloat16 kernels take head sizes that are multiples of 16 "
                             f"and widths that are multiples of 8 (here {self.head_dim} and {self.width}); "
                             "the float32 path takes this model")
        t = self.stored == "in_out"
        self.w_qkv = runtime.matrix(get(self.qkv_name + ".weight"), transpose=t)
        self.w_out = runtime.matrix(get(self.out_name + ".weight"), transpose=t)
        if self.bias:
            self.b_qkv = runtime.vector(get(self.qkv_name + ".bias"))
            self.b_out = runtime.vector(get(self.out_name + ".bias"))

    def stream_weights(self):
        return [self.w_qkv, self.w_out]

    def cache_need(self):
        return CacheNeed("window" if self.window > 0 else "full", self.kv_heads, self.head_dim, self.window)

    def forward(self, ctx, h, residual, app):
        ops = ctx.ops
        qkv = ops.linear(h, self.w_qkv, self.b_qkv, out_dtype=ctx.dtype)
        ctx.position.apply_qk(ctx, qkv, self.n_heads, self.kv_heads, self.head_dim)
        a = ops.attention(qkv, app.cache, ctx.plan, self.n_heads, self.kv_heads, self.head_dim, self.scale,
                          self.window, out_dtype=ctx.dtype, store=app.writes_cache)
        return ops.linear(a, self.w_out, self.b_out, residual=residual)


register_part("mixer", "causal_attention", CausalAttention)
