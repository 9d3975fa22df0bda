"""The matrix memory of the xLSTM (mLSTM) as a mixer with per-sequence state and no cache
(Beck et al., "xLSTM: Extended Long Short-Term Memory").

Per head: q = W_q h * dim^(-1/2), k = W_k h (dim values each), v = W_v h (vdim values), a log input
gate i = cap * tanh((w_i . h + b_i) / cap) and a log forget gate f = logsigmoid(cap * tanh((w_f . h +
b_f) / cap)).  With a memory S of dim x vdim values, a normaliser n of dim values and a running
maximum m, all starting at zero:

    m_t = max(f_t + m_(t-1), i_t)
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T      n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + floor)

Each head's o is divided by its root mean square, the heads laid end to end are multiplied by a gain
and by sigmoid(W_g h), and projected out.  The gates, the maxima, the recurrence and its state, and
the norm are float32 in every mode; the projections q | k | v | g are in the compute type.

What a sequence carries from step to step: S, n and m of every head (`StateNeed`s "S", "n", "m").
"""
from __future__ import annotations

from .base import Mixer, StateNeed, WeightSpec, register_part

DENOMINATOR_FLOOR = 1e-6     # added to the read-out's denominator


class MLSTM(Mixer):

    def __init__(self, prefix: str, width: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 q: str = "q", k: str = "k", v: str = "v", gate: str = "g", input_gate: str = "i", forget_gate: str = "f",
                 bias_suffix: str = ".b", norm: str = "norm", out: str = "o", init_std: float = 0.02,
                 out_init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.heads, self.dim, self.vdim = int(width), int(heads), int(dim), int(vdim)
        self.cap, self.eps = float(gate_cap), float(eps)
        if self.heads <= 0 or not 1 <= self.dim <= 256 or not 1 <= self.vdim <= 65536:
            raise ValueError(f"mlstm {prefix!r}: {self.heads} heads of {self.dim} and {self.vdim} (key size in [1, 256])")
        if self.cap < 0:
            raise ValueError(f"mlstm {prefix!r}: gate_cap = {self.cap} is negative")
        self.qk, self.inner = self.heads * self.dim, self.heads * self.vdim
        self.proj_width = 2 * self.qk + 2 * self.inner                   # q | k | v | g
        self.names = {n: prefix + s for n, s in dict(q=q, k=k, v=v, gate=gate, i=input_gate, f=forget_gate, norm=norm,
                                                     out=out).items()}
        self.bias_suffix = bias_suffix
        self.init_std, self.out_init_std = init_std, out_init_std
        self.w_in = self.w_gates = self.w_out = None

    def weight_specs(self):
        n, d = self.names, self.width
        return [WeightSpec(n["q"], (self.qk, d), std=self.init_std), WeightSpec(n["k"], (self.qk, d), std=self.init_std),
                WeightSpec(n["v"], (self.inner, d), std=self.init_std), WeightSpec(n["gate"], (self.inner, d), std=self.init_std),
                WeightSpec(n["out"], (d, self.inner), std=self.out_init_std),
                WeightSpec(n["norm"], (self.inner,), mean=1.0, std=0.1),
                WeightSpec(n["i"], (self.heads, d), std=self.init_std), WeightSpec(n["i"] + self.bias_suffix, (self.heads,), mean=-1.0, std=1.0),
                WeightSpec(n["f"], (self.heads, d), std=self.init_std), WeightSpec(n["f"] + self.bias_suffix, (self.heads,), mean=3.0, std=1.0)]

    def load(self, get, runtime):
        import torch
        n = self.names
        w = torch.cat([runtime.matrix(get(n[k])) for k in ("q", "k", "v", "gate")])
        # rows of zeros up to a multiple of 8: every row of the projection's output then starts on 16 bytes
        self.proj_stride = -(-self.proj_width // 8) * 8
        if self.proj_stride != self.proj_width:
            w = torch.cat([w, torch.zeros((self.proj_stride - self.proj_width, self.width), dtype=w.dtype, device=w.device)])
        self.w_in = w.contiguous()
        self.w_gates = torch.cat([runtime.matrix(get(n["i"])), runtime.matrix(get(n["f"]))]).contiguous()
        self.b_gates = torch.cat([runtime.vector(get(n["i"] + self.bias_suffix)), runtime.vector(get(n["f"] + self.bias_suffix))]).contiguous()
        self.w_out = runtime.matrix(get(n["out"]))
        self.norm_w = runtime.vector(get(n["norm"]))

    def stream_weights(self):
        return [self.w_in, self.w_out]

    def state_need(self):
        return {"S": StateNeed((self.heads, self.dim, self.vdim)), "n": StateNeed((self.heads, self.dim)),
                "m": StateNeed((self.heads,))}

    def _mix(self, ctx, h, app):
        ops = ctx.ops
        proj = ops.linear(h, self.w_in, None, out_dtype=ctx.dtype)                      # [T, q | k | v | g (| 0)]
        gates = ops.mlstm_gates(h, self.w_gates, self.b_gates, self.heads, self.cap)    # float32 [T, i | f]
        o = ops.mlstm_scan(proj, 0, self.qk, 2 * self.qk, gates, app.state, ctx.plan, self.heads, self.dim, self.vdim,
                           DENOMINATOR_FLOOR)
        return ops.gated_group_norm(o, proj, 2 * self.qk + self.inner, self.norm_w, self.heads, self.eps, ctx.dtype,
                                    gate_first=False, gate="sigmoid")

    def forward(self, ctx, h, residual, app):
        return ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, residual=residual)

    def branches(self, ctx, h, app):
        import torch
        return [(ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, out_dtype=torch.float32), 1.0)]


register_part("mixer", "mlstm", MLSTM)
