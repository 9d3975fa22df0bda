"""Norms.

LayerNorm with bias as ember.cpp computes it: mean and biased variance in two passes,
`(x - mean) * 1/sqrt(var + eps) * w + b` (graph_ir.cpp:2421-2439; the CUDA kernel
graph_ir_cuda.cu:47-65 accumulates both sums in double).  Here the statistics are in float32 on
the residual stream, which is float32 in every mode.

RMS norm: `x / sqrt(mean(x^2) + eps) * (offset + w)`, the statistics in float32 too.  `offset` is
0 for a gain stored as it is used and 1 for a gain stored as its distance from one.  No bias.
"""
from __future__ import annotations

from .base import Norm, WeightSpec, plain_branches, register_part


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


class RMSNorm(Norm):

    def __init__(self, prefix: str, width: int, eps: float, weight: str = "weight", offset: float = 0.0,
                 init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.eps, self.offset = int(width), float(eps), float(offset)
        self.weight_name, self.init_std = prefix + weight, init_std
        self.w = None

    def weight_specs(self):
        # random-weights mode: the gain as used is 1 + N(0, std)
        return [WeightSpec(self.weight_name, (self.width,), mean=1.0 - self.offset, std=self.init_std)]

    def load(self, get, runtime):
        self.w = runtime.vector(get(self.weight_name))

    def forward(self, ctx, x, out_dtype):
        return ctx.ops.rmsnorm(x, self.w, self.eps, out_dtype, offset=self.offset)

    def add_normed(self, ctx, x, branches):
        """One launch: the weighted sum of the branches, its norm, and the sum with the stream."""
        return ctx.ops.add_normed(x, plain_branches(ctx, branches), self.w, self.eps, offset=self.offset)


class LayerScale(Norm):
    """A gain per channel and nothing else: `x * w`.  In the place of a norm after a sublayer (the `sandwich`
    arrangement's `after_mixer` / `after_ffn`) it is the layer scale of a pre-norm block: the stream gets
    `x + w * (sum of the sublayer's branches)`, in one launch, branches with norms of their own included."""

    def __init__(self, prefix: str, width: int, weight: str = "weight", eps: float = 0.0, init_mean: float = 1.0,
                 init_std: float = 0.1):
        super().__init__(prefix)
        self.width, self.eps = int(width), float(eps)       # eps: for branches that are normed one by one and name none
        self.weight_name, self.init_mean, self.init_std = prefix + weight, init_mean, init_std
        self.w = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.width,), mean=self.init_mean, std=self.init_std)]

    def load(self, get, runtime):
        self.w = runtime.vector(get(self.weight_name))

    def forward(self, ctx, x, out_dtype):
        return (x * self.w).to(out_dtype)

    def add_normed(self, ctx, x, branches):
        eps = {b[2][1] for b in branches if len(b) > 2 and b[2] is not None}
        if len(eps) > 1:        # (one launch takes one eps: norms of different eps are carried out first)
            branches, eps = plain_branches(ctx, branches), set()
        flat = [(b[0], b[1], b[2][0] if len(b) > 2 and b[2] is not None else None) for b in branches]
        return ctx.ops.add_branches(x, flat, self.w, eps.pop() if eps else self.eps)


register_part("norm", "layernorm", LayerNorm)
register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layer_scale", LayerScale)
