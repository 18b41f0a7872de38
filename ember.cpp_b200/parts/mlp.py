"""Dense feed-forward: up projection, activation, down projection, added to the residual stream.

ember.cpp's GPT-2 block: `u = h Wup^T + b; u = gelu(u); f = u Wdown^T + b; x = x + f`
(graph_ir.cpp:743-746, 754-756) with GELU in its tanh form
`0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3)))` or its erf form `0.5 v (1 + erf(v / sqrt 2))`
(graph_ir.cpp:2471-2481; graph_ir_cuda.cu:230-242).
"""
from __future__ import annotations

from .base import FeedForward, WeightSpec, register_part

ACTIVATIONS = ("gelu_tanh", "gelu_erf")


class DenseFeedForward(FeedForward):

    def __init__(self, prefix: str, width: int, inner: int, activation: str, up: str = "c_fc", down: str = "c_proj",
                 stored: str = "in_out", bias: bool = True, init_std: float = 0.02, down_init_std: float = 0.02,
                 bias_init_std: float = 0.01):
        super().__init__(prefix)
        if activation not in ACTIVATIONS:
            raise ValueError(f"feed-forward {prefix!r}: activation {activation!r} is not one of {ACTIVATIONS}")
        if stored not in ("in_out", "out_in"):
            raise ValueError(f"feed-forward {prefix!r}: stored = {stored!r}")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.up_name, self.down_name, self.stored, self.bias = prefix + up, prefix + down, stored, bias
        self.init_std, self.down_init_std, self.bias_init_std = init_std, down_init_std, bias_init_std
        self.w_up = self.b_up = self.w_down = self.b_down = None

    def _shape(self, n_in, n_out):
        return (n_in, n_out) if self.stored == "in_out" else (n_out, n_in)

    def weight_specs(self):
        specs = [WeightSpec(self.up_name + ".weight", self._shape(self.width, self.inner), std=self.init_std),
                 WeightSpec(self.down_name + ".weight", self._shape(self.inner, self.width), std=self.down_init_std)]
        if self.bias:
            specs += [WeightSpec(self.up_name + ".bias", (self.inner,), std=self.bias_init_std),
                      WeightSpec(self.down_name + ".bias", (self.width,), std=self.bias_init_std)]
        return specs

    def load(self, get, runtime):
        import torch
        if runtime.dtype == torch.bfloat16 and (self.inner % 8 or self.width % 8):
            raise ValueError(f"feed-forward {self.prefix!r}: the bfloat16 kernels take widths that are multiples of 8 "
                             f"(rows of 16 bytes; here width {self.width}, inner {self.inner}); the float32 path takes this model")
        t = self.stored == "in_out"
        self.w_up = runtime.matrix(get(self.up_name + ".weight"), transpose=t)
        self.w_down = runtime.matrix(get(self.down_name + ".weight"), transpose=t)
        if self.bias:
            self.b_up = runtime.vector(get(self.up_name + ".bias"))
            self.b_down = runtime.vector(get(self.down_name + ".bias"))

    def stream_weights(self):
        return [self.w_up, self.w_down]

    def forward(self, ctx, h, residual):
        warm = getattr(ctx.ops, "warm", None)
        if warm is not None:
            warm(self.w_down)  # a hint: the second product's weights can be on their way during the first
        u = ctx.ops.linear(h, self.w_up, self.b_up, act=self.activation, out_dtype=ctx.dtype)
        return ctx.ops.linear(u, self.w_down, self.b_down, residual=residual)


register_part("ffn", "dense", DenseFeedForward)
