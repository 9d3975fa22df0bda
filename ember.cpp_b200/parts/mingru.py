"""minGRU as a mixer with per-sequence state and no cache (Feng et al., "Were RNNs All We Needed?"):
a gated recurrence whose gate and candidate read the current token alone.

    z_t = sigmoid(W_z h_t + b_z)      u_t = W_x h_t + b_x      c_t = u_t + 1/2 where u_t >= 0, sigmoid(u_t) where u_t < 0
    S_t = (1 - z_t) S_(t-1) + z_t c_t   (element by element, S starts at zero)      out_t = W_o (S_t * silu(W_g h_t))

One stacked projection makes z | x | g; it is left in float32 in every mode, because the gate and the
candidate enter the recurrence.  Gates, candidates and the state are float32; the gated state goes into the
output projection in the compute type.

What a sequence carries from step to step: S (`StateNeed` of `width` values).
"""
from __future__ import annotations

from .base import Mixer, StateNeed, WeightSpec, register_part


class MinGRU(Mixer):

    def __init__(self, prefix: str, width: int, inner: int, gate: str = "z", candidate: str = "x", out_gate: str = "g",
                 bias_suffix: str = ".b", out: str = "o", init_std: float = 0.02, out_init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.inner = int(width), int(inner)
        if self.inner <= 0:
            raise ValueError(f"mingru {prefix!r}: a state of {self.inner} values")
        self.names = {n: prefix + s for n, s in dict(z=gate, x=candidate, g=out_gate, out=out).items()}
        self.bias_suffix = bias_suffix
        self.init_std, self.out_init_std = init_std, out_init_std
        self.w_in = self.w_out = None

    def weight_specs(self):
        n, d = self.names, self.width
        return [WeightSpec(n["z"], (self.inner, d), std=self.init_std), WeightSpec(n["z"] + self.bias_suffix, (self.inner,), std=1.0),
                WeightSpec(n["x"], (self.inner, d), std=self.init_std), WeightSpec(n["x"] + self.bias_suffix, (self.inner,), std=0.5),
                WeightSpec(n["g"], (self.inner, d), std=self.init_std),
                WeightSpec(n["out"], (d, self.inner), std=self.out_init_std)]

    def load(self, get, runtime):
        import torch
        n = self.names
        # every part of z | x | g starts on a multiple of 8 columns (rows of zeros between them where the size is none)
        self.part = -(-self.inner // 8) * 8
        pieces = []
        for k in ("z", "x", "g"):
            w = runtime.matrix(get(n[k]))
            if self.part != self.inner:
                w = torch.cat([w, torch.zeros((self.part - self.inner, self.width), dtype=w.dtype, device=w.device)])
            pieces.append(w)
        self.w_in = torch.cat(pieces).contiguous()
        self.b_z = runtime.vector(get(n["z"] + self.bias_suffix))
        self.b_x = runtime.vector(get(n["x"] + self.bias_suffix))
        self.w_out = runtime.matrix(get(n["out"]))

    def stream_weights(self):
        return [self.w_in, self.w_out]

    def state_need(self):
        return StateNeed((self.inner,))

    def _mix(self, ctx, h, app):
        import torch
        ops = ctx.ops
        proj = ops.linear(h, self.w_in, None, out_dtype=torch.float32)                  # float32 [T, z | x | g]
        return ops.mingru(proj, 0, self.part, 2 * self.part, self.b_z, self.b_x, app.state, ctx.plan, self.inner, ctx.dtype)

    def forward(self, ctx, h, residual, app):
        return ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, residual=residual)

    def branches(self, ctx, h, app):
        import torch
        return [(ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, out_dtype=torch.float32), 1.0)]


register_part("mixer", "mingru", MinGRU)
