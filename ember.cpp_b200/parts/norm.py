"""Norms.

LayerNorm with bias as ember.cpp computes it: mean and biased variance in two passes,
`(x - mean) * 1/sqrt(var + eps) * w + b` (graph_ir.cpp:2421-2439; the CUDA kernel
graph_ir_cuda.cu:47-65 accumulates both sums in double).  Here the statistics are in float32 on
the residual stream, which is float32 in every mode.
"""
from __future__ import annotations

from .base import Norm, WeightSpec, register_part


class LayerNorm(Norm):

    def __init__(self, prefix: str, width: int, eps: float, weight: str = "weight", bias: str = "bias"):
        super().__init__(prefix)
        self.width, self.eps = int(width), float(eps)
        self.weight_name, self.bias_name = prefix + weight, prefix + bias
        self.w = self.b = None

    def weight_specs(self):
        # random-weights mode: gamma = 1 + N(0, 0.02), beta = N(0, 0.02)
        return [WeightSpec(self.weight_name, (self.width,), mean=1.0, std=0.02),
                WeightSpec(self.bias_name, (self.width,), mean=0.0, std=0.02)]

    def load(self, get, runtime):
        self.w = runtime.vector(get(self.weight_name))
        self.b = runtime.vector(get(self.bias_name))

    def forward(self, ctx, x, out_dtype):
        return ctx.ops.layernorm(x, self.w, self.b, self.eps, out_dtype)


register_part("norm", "layernorm", LayerNorm)
