"""Dense feed-forward: up projection, activation, down projection, added to the residual stream.

ember.cpp's GPT-2 block: `u = h Wup^T + b; u = gelu(u); f = u Wdown^T + b; x = x + f`
(graph_ir.cpp:743-746, 754-756) with GELU in its tanh form
`0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3)))` or its erf form `0.5 v (1 + erf(v / sqrt 2))`
(graph_ir.cpp:2471-2481; graph_ir_cuda.cu:230-242).

Gated feed-forward: two projections of the input side by side, `y = act(g) * u`, then the down
projection.  `silu`: act(g) = g * sigmoid(g), the usual gated layer.  `clamped_sigmoid`: g is first
capped from above at `limit` and u held within +-`limit`, then y = g * sigmoid(alpha * g) * (u + shift).
The two matrices are laid one under the other at load, so a step makes one product for both.
"""
from __future__ import annotations

from .base import FeedForward, WeightSpec, register_part

ACTIVATIONS = ("gelu_tanh", "gelu_erf", "relu2")     # relu2: the square of relu


class DenseFeedForward(FeedForward):

    def __init__(self, prefix: str, width: int, inner: int, activation: str, up: str = "c_fc", down: str = "c_proj",
                 stored: str = "in_out", bias: bool = True, init_std: float = 0.02, down_init_std: float = 0.02,
                 bias_init_std: float = 0.01, suffix: str = ".weight", any_size: bool = False):
        super().__init__(prefix)
        self.any_size = any_size  # True: widths that are no multiples of 8 are left to the slower products in bfloat16
        self.suffix = suffix      # what follows a matrix's name in the checkpoint ("" for names without one)
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
        specs = [WeightSpec(self.up_name + self.suffix, self._shape(self.width, self.inner), std=self.init_std),
                 WeightSpec(self.down_name + self.suffix, self._shape(self.inner, self.width), std=self.down_init_std)]
        if self.bias:
            specs += [WeightSpec(self.up_name + ".bias", (self.inner,), std=self.bias_init_std),
                      WeightSpec(self.down_name + ".bias", (self.width,), std=self.bias_init_std)]
        return specs

    def load(self, get, runtime):
        import torch
        if runtime.dtype == torch.bfloat16 and (self.inner % 8 or self.width % 8) and not self.any_size:
            raise ValueError(f"feed-forward {self.prefix!r}: the bfloat16 kernels take widths that are multiples of 8 "
                             f"(rows of 16 bytes; here width {self.width}, inner {self.inner}); the float32 path takes this model")
        t = self.stored == "in_out"
        self.w_up = runtime.matrix(get(self.up_name + self.suffix), transpose=t)
        self.w_down = runtime.matrix(get(self.down_name + self.suffix), transpose=t)
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

    def branches(self, ctx, h):
        import torch
        u = ctx.ops.linear(h, self.w_up, self.b_up, act=self.activation, out_dtype=ctx.dtype)
        return [(ctx.ops.linear(u, self.w_down, self.b_down, out_dtype=torch.float32), 1.0)]


GATES = ("silu", "clamped_sigmoid")


class GatedFeedForward(FeedForward):

    def __init__(self, prefix: str, width: int, inner: int, activation: str = "silu", limit: float = 0.0,
                 alpha: float = 1.0, shift: float = 0.0, gate: str = "gate", up: str = "up", down: str = "down",
                 suffix: str = ".weight", init_std: float = 0.02, down_init_std: float = 0.02):
        super().__init__(prefix)
        if activation not in GATES:
            raise ValueError(f"feed-forward {prefix!r}: activation {activation!r} is not one of {GATES}")
        if activation == "clamped_sigmoid" and not limit > 0:
            raise ValueError(f"feed-forward {prefix!r}: limit = {limit} must be positive")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.gate_name, self.up_name, self.down_name = (prefix + n + suffix for n in (gate, up, down))
        self.init_std, self.down_init_std = init_std, down_init_std
        self.w_gate_up = self.w_down = None

    def weight_specs(self):
        return [WeightSpec(self.gate_name, (self.inner, self.width), std=self.init_std),
                WeightSpec(self.up_name, (self.inner, self.width), std=self.init_std),
                WeightSpec(self.down_name, (self.width, self.inner), std=self.down_init_std)]

    def load(self, get, runtime):
        import torch
        self.w_gate_up = torch.cat([runtime.matrix(get(self.gate_name)), runtime.matrix(get(self.up_name))]).contiguous()
        self.w_down = runtime.matrix(get(self.down_name))

    def stream_weights(self):
        return [self.w_gate_up, self.w_down]

    def _inner(self, ctx, h):
        gu = ctx.ops.linear(h, self.w_gate_up, None, out_dtype=ctx.dtype)          # [T, gate | up]
        return ctx.ops.gated_act(gu, self.activation, self.limit, self.alpha, self.shift)

    def forward(self, ctx, h, residual):
        return ctx.ops.linear(self._inner(ctx, h), self.w_down, None, residual=residual)

    def branches(self, ctx, h):
        import torch
        return [(ctx.ops.linear(self._inner(ctx, h), self.w_down, None, out_dtype=torch.float32), 1.0)]


register_part("ffn", "dense", DenseFeedForward)
register_part("ffn", "gated", GatedFeedForward)
