"""Gated linear attention as a mixer with per-sequence state and no cache (Yang, Wang, Shen, Panda, Kim,
"Gated Linear Attention Transformers with Hardware-Efficient Training").

Per head: q = W_q h * dim^(-1/2), k = W_k h (dim values each), v = W_v h (vdim values), and a decay for
every key channel, alpha = sigmoid(z)^(1/tau) with z = W_a2 (W_a1 h) + b a product of low rank.  With a
state S of dim x vdim float32 values that starts at zero:

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t

Each head's o is divided by its root mean square and multiplied by a gain of vdim values that the heads
share; the heads laid end to end are multiplied by silu(W_g h) and projected out.  The low-rank product's
second half, the decays, the recurrence and its state, and the norm are float32 in every mode; the
projections q | k | v | g | a1 are one product in the compute type.

What a sequence carries from step to step: S of every head (`StateNeed` "S").
"""
from __future__ import annotations

from .base import Mixer, StateNeed, WeightSpec, register_part


class GatedLinearAttention(Mixer):

    def __init__(self, prefix: str, width: int, heads: int, dim: int, vdim: int, tau: float, eps: float,
                 q: str = "q", k: str = "k", v: str = "v", gate: str = "g", decay_in: str = "a1", decay_out: str = "a2",
                 bias_suffix: str = ".b", norm: str = "norm", out: str = "o", rank: int = 16, init_std: float = 0.02,
                 out_init_std: float = 0.02):
        """rank: of the decay's two-step product in random-weights mode; a checkpoint's tensors give their own."""
        super().__init__(prefix)
        self.width, self.heads, self.dim, self.vdim = int(width), int(heads), int(dim), int(vdim)
        self.tau, self.eps = float(tau), float(eps)
        if self.heads <= 0 or not 1 <= self.dim <= 256 or not 1 <= self.vdim <= 65536:
            raise ValueError(f"gated linear attention {prefix!r}: {self.heads} heads of {self.dim} and {self.vdim} (key size in [1, 256])")
        if not self.tau > 0:
            raise ValueError(f"gated linear attention {prefix!r}: tau = {self.tau} must be positive")
        self.qk, self.inner = self.heads * self.dim, self.heads * self.vdim
        self.names = {n: prefix + s for n, s in dict(q=q, k=k, v=v, gate=gate, a1=decay_in, a2=decay_out, norm=norm,
                                                     out=out).items()}
        self.bias_suffix, self.rank = bias_suffix, int(rank)
        self.init_std, self.out_init_std = init_std, out_init_std
        self.w_in = self.w_out = None

    def weight_specs(self):
        n, d, r = self.names, self.width, self.rank
        return [WeightSpec(n["q"], (self.qk, d), std=self.init_std), WeightSpec(n["k"], (self.qk, d), std=self.init_std),
                WeightSpec(n["v"], (self.inner, d), std=self.init_std), WeightSpec(n["gate"], (self.inner, d), std=self.init_std),
                WeightSpec(n["out"], (d, self.inner), std=self.out_init_std),
                WeightSpec(n["norm"], (self.vdim,), mean=1.0, std=0.1),
                WeightSpec(n["a1"], (r, d), std=self.init_std, free=(0,)), WeightSpec(n["a2"], (self.qk, r), std=0.5, free=(1,)),
                WeightSpec(n["a2"] + self.bias_suffix, (self.qk,), mean=2.0, std=1.0)]

    def load(self, get, runtime):
        import torch
        n = self.names
        parts = [runtime.matrix(get(n[k])) for k in ("q", "k", "v", "gate", "a1")]
        self.rank = parts[-1].shape[0]
        if self.rank > 256 or get(n["a2"]).shape[1] != self.rank:
            raise ValueError(f"gated linear attention {self.prefix!r}: the decay's two matrices meet in {self.rank} and "
                             f"{get(n['a2']).shape[1]} values (one rank of at most 256)")
        w = torch.cat(parts)
        self.proj_width = w.shape[0]
        # rows of zeros up to a multiple of 8: every row of the projection's output then starts on 16 bytes
        pad = -w.shape[0] % 8
        if pad:
            w = torch.cat([w, torch.zeros((pad, self.width), dtype=w.dtype, device=w.device)])
        self.w_in = w.contiguous()
        self.w_out = runtime.matrix(get(n["out"]))
        self.w_a2 = runtime.vector(get(n["a2"])).t().contiguous()                 # float32 [rank, heads * dim]: transposed
        self.b_a2 = runtime.vector(get(n["a2"] + self.bias_suffix))
        self.norm_w = runtime.vector(get(n["norm"])).repeat(self.heads).contiguous()     # the heads share the gain

    def stream_weights(self):
        return [self.w_in, self.w_out]

    def state_need(self):
        return {"S": StateNeed((self.heads, self.dim, self.vdim))}

    def _mix(self, ctx, h, app):
        ops = ctx.ops
        proj = ops.linear(h, self.w_in, None, out_dtype=ctx.dtype)                       # [T, q | k | v | g | a1 (| 0)]
        g_col = 2 * self.qk + self.inner
        z = ops.low_rank_out(proj, g_col + self.inner, self.w_a2, self.b_a2, "none")      # float32 [T, heads * dim]
        o = ops.gla_scan(proj, 0, self.qk, 2 * self.qk, z, self.tau, app.state["S"], ctx.plan, self.heads, self.dim, self.vdim)
        return ops.gated_group_norm(o, proj, g_col, self.norm_w, self.heads, self.eps, ctx.dtype, gate_first=False)

    def forward(self, ctx, h, residual, app):
        return ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, residual=residual)

    def branches(self, ctx, h, app):
        import torch
        return [(ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, out_dtype=torch.float32), 1.0)]


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
