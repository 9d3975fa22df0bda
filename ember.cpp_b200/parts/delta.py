"""The gated delta rule as a mixer with per-sequence state and no cache.

One input projection makes, side by side, q | k | v | gate | b | a.  q, k and v pass a short
causal convolution over the sequence (one filter per channel, the last tap on the current token,
zeros before the sequence's start, no bias) and silu.  Per head q and k become unit vectors
(x / sqrt(sum x^2 + 1e-6)), q times dim^(-1/2); head h reads the q and k of key head
h // (heads / kv_heads).  Per head, with a state S of dim x vdim float32 values that starts at
zero (Yang, Kautz, Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta Rule"):

    beta_t = sigmoid(b_t)        g_t = exp(-exp(A_log) * softplus(a_t + dt_bias))
    S  <- g_t S;    u = beta_t (v_t - S^T k_t);    S <- S + k_t u^T;    o_t = S^T q_t

so the read-out sees the token's own write.  o is divided by its root mean square over a head,
multiplied by a gain of vdim values that the heads share and by silu(gate), and projected out.
The unit vectors, beta, the decays, the recurrence and its state, and the norm are float32 in
every mode; the projection and the convolution with its silu are in the compute type.

What a sequence carries from step to step: S of every head, and the last `conv` - 1 rows that
entered the convolution (`StateNeed`s "S" and "conv").
"""
from __future__ import annotations

from .base import Mixer, StateNeed, WeightSpec, register_part

UNIT_EPS = 1e-6     # inside the root of the unit vectors' length


class GatedDeltaRule(Mixer):

    def __init__(self, prefix: str, width: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, eps: float,
                 q: str = "q", k: str = "k", v: str = "v", gate: str = "g", beta: str = "b", step: str = "a",
                 conv_suffix: str = ".conv", dt_bias: str = "dt_bias", a_log: str = "A_log", norm: str = "norm",
                 out: str = "o", init_std: float = 0.02, out_init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.heads, self.kv_heads = int(width), int(heads), int(kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(dim), int(vdim), int(conv), float(eps)
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"delta rule {prefix!r}: {self.heads} heads are not a multiple of {self.kv_heads} key heads")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"delta rule {prefix!r}: a convolution of {self.taps} taps is not in [1, 16]")
        if not (1 <= self.dim <= 1024 and 1 <= self.vdim <= 1024):
            raise ValueError(f"delta rule {prefix!r}: head sizes {self.dim} and {self.vdim} are not in [1, 1024]")
        self.qk, self.inner = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk + self.inner                 # q | k | v, what the convolution sees
        self.proj_width = self.channels + self.inner + 2 * self.heads
        self.names = {n: prefix + s for n, s in dict(q=q, k=k, v=v, gate=gate, beta=beta, step=step, dt_bias=dt_bias,
                                                     a_log=a_log, norm=norm, out=out).items()}
        self.conv_suffix = conv_suffix
        self.init_std, self.out_init_std = init_std, out_init_std
        self.w_in = self.w_out = None

    def weight_specs(self):
        n, d = self.names, self.width
        return [WeightSpec(n["q"], (self.qk, d), std=self.init_std), WeightSpec(n["q"] + self.conv_suffix, (self.qk, self.taps), std=0.3),
                WeightSpec(n["k"], (self.qk, d), std=self.init_std), WeightSpec(n["k"] + self.conv_suffix, (self.qk, self.taps), std=0.3),
                WeightSpec(n["v"], (self.inner, d), std=self.init_std), WeightSpec(n["v"] + self.conv_suffix, (self.inner, self.taps), std=0.3),
                WeightSpec(n["beta"], (self.heads, d), std=self.init_std),
                WeightSpec(n["a_log"], (self.heads,), mean=-0.5, std=0.5),
                WeightSpec(n["norm"], (self.vdim,), mean=1.0, std=0.1),
                WeightSpec(n["step"], (self.heads, d), std=self.init_std),
                WeightSpec(n["dt_bias"], (self.heads,), mean=-1.0, std=0.5),
                WeightSpec(n["gate"], (self.inner, d), std=self.init_std),
                WeightSpec(n["out"], (d, self.inner), std=self.out_init_std)]

    def load(self, get, runtime):
        import torch
        n = self.names
        w = torch.cat([runtime.matrix(get(n[k])) for k in ("q", "k", "v", "gate", "beta", "step")])
        # rows of zeros up to a multiple of 8: every row of the projection's output then starts on 16 bytes
        self.proj_stride = -(-self.proj_width // 8) * 8
        if self.proj_stride != self.proj_width:
            w = torch.cat([w, torch.zeros((self.proj_stride - self.proj_width, self.width), dtype=w.dtype, device=w.device)])
        self.w_in = w.contiguous()
        self.w_out = runtime.matrix(get(n["out"]))
        self.conv_w = torch.cat([runtime.vector(get(n[k] + self.conv_suffix)) for k in ("q", "k", "v")]).contiguous()
        self.conv_b = torch.zeros(self.channels, dtype=torch.float32, device=self.conv_w.device)
        self.dt_bias = runtime.vector(get(n["dt_bias"]))
        self.a_log = runtime.vector(get(n["a_log"]))
        self.norm_w = runtime.vector(get(n["norm"])).repeat(self.heads).contiguous()     # the heads share the gain

    def stream_weights(self):
        return [self.w_in, self.w_out]

    def state_need(self):
        need = {"S": StateNeed((self.heads, self.dim, self.vdim))}
        if self.taps > 1:
            need["conv"] = StateNeed((self.taps - 1, self.channels))       # the rows before the step's first, oldest first
        return need

    def _mix(self, ctx, h, app):
        ops = ctx.ops
        proj = ops.linear(h, self.w_in, None, out_dtype=ctx.dtype)                     # [T, q k v | gate | b | a (| 0)]
        qkv = ops.conv_silu(proj, 0, self.channels, self.conv_w, self.conv_b, app.state.get("conv"), ctx.plan)
        gate_col = self.channels
        o = ops.delta_rule(qkv, proj, gate_col + self.inner, gate_col + self.inner + self.heads, self.a_log, self.dt_bias,
                           app.state["S"], ctx.plan, self.heads, self.kv_heads, self.dim, self.vdim, UNIT_EPS)
        return ops.gated_group_norm(o, proj, gate_col, self.norm_w, self.heads, self.eps, ctx.dtype, gate_first=False)

    def forward(self, ctx, h, residual, app):
        return ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, residual=residual)

    def branches(self, ctx, h, app):
        import torch
        return [(ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, out_dtype=torch.float32), 1.0)]


register_part("mixer", "gated_delta_rule", GatedDeltaRule)


class GeneralizedDeltaRule(Mixer):
    """The delta rule with a decay and a removal rate for every key channel (the state update of RWKV-7:
    Peng et al., "RWKV-7 'Goose' with Expressive Dynamic State Evolution").

    Per head r = W_r h, k = W_k h, v = W_v h (dim values each), a decay
    w = exp(-decay_coef * sigmoid(W_w2 tanh(W_w1 h) + w0)) and a removal rate a = sigmoid(W_a h + b_a) for
    every key channel.  With the unit key u = k / sqrt(sum k^2 + 1e-6) and a state S of dim x dim float32
    values that starts at zero:

        S_t = diag(w_t) S_(t-1) - (a_t * u_t)(u_t^T S_(t-1)) + k_t v_t^T        o_t = S_t^T r_t

    both of the first two terms reading the state of the token before.  Each head's o is divided by its
    root mean square, the heads laid end to end are multiplied by a gain of that whole size and by
    sigmoid(W_g h), and projected out.  The decay's second product, the decays and rates, the unit keys,
    the recurrence and its state, and the norm are float32 in every mode; r | k | v | g | a | w1 are one
    product in the compute type.  What a sequence carries: S of every head (`StateNeed` "S")."""

    def __init__(self, prefix: str, width: int, heads: int, dim: int, eps: float, decay_coef: float,
                 r: str = "r", k: str = "k", v: str = "v", gate: str = "g", rate: str = "a", decay_in: str = "w1",
                 decay_out: str = "w2", decay_bias: str = "w0", bias_suffix: str = ".b", norm: str = "norm", out: str = "o",
                 rank: int = 16, init_std: float = 0.02, out_init_std: float = 0.02):
        """rank: of the decay's two-step product in random-weights mode; a checkpoint's tensors give their own."""
        super().__init__(prefix)
        self.width, self.heads, self.dim = int(width), int(heads), int(dim)
        self.eps, self.decay_coef, self.rank = float(eps), float(decay_coef), int(rank)
        if self.heads <= 0 or not 1 <= self.dim <= 256:
            raise ValueError(f"generalized delta rule {prefix!r}: {self.heads} heads of {self.dim} (head size in [1, 256])")
        self.inner = self.heads * self.dim
        self.names = {n: prefix + s for n, s in dict(r=r, k=k, v=v, gate=gate, a=rate, w1=decay_in, w2=decay_out,
                                                     w0=decay_bias, norm=norm, out=out).items()}
        self.bias_suffix = bias_suffix
        self.init_std, self.out_init_std = init_std, out_init_std
        self.w_in = self.w_out = None

    def weight_specs(self):
        n, d, m = self.names, self.width, self.inner
        return [WeightSpec(n[key], (m, d), std=self.init_std) for key in ("r", "k", "v", "gate", "a")] + [
            WeightSpec(n["a"] + self.bias_suffix, (m,), std=1.0),
            WeightSpec(n["w1"], (self.rank, d), std=self.init_std, free=(0,)),
            WeightSpec(n["w2"], (m, self.rank), std=0.5, free=(1,)),
            WeightSpec(n["w0"], (m,), std=1.0),
            WeightSpec(n["norm"], (m,), mean=1.0, std=0.1),
            WeightSpec(n["out"], (d, m), std=self.out_init_std)]

    def load(self, get, runtime):
        import torch
        n = self.names
        parts = [runtime.matrix(get(n[key])) for key in ("r", "k", "v", "gate", "a", "w1")]
        self.rank = parts[-1].shape[0]
        if self.rank > 256 or get(n["w2"]).shape[1] != self.rank:
            raise ValueError(f"generalized delta rule {self.prefix!r}: the decay's two matrices meet in {self.rank} and "
                             f"{get(n['w2']).shape[1]} values (one rank of at most 256)")
        w = torch.cat(parts)
        pad = -w.shape[0] % 8      # rows of zeros: every row of the projection's output starts on 16 bytes
        if pad:
            w = torch.cat([w, torch.zeros((pad, self.width), dtype=w.dtype, device=w.device)])
        self.w_in = w.contiguous()
        self.w_out = runtime.matrix(get(n["out"]))
        self.w_w2 = runtime.vector(get(n["w2"])).t().contiguous()  # float32 [rank, heads * dim]: transposed
        self.w0 = runtime.vector(get(n["w0"]))
        self.b_a = runtime.vector(get(n["a"] + self.bias_suffix))
        self.norm_w = runtime.vector(get(n["norm"]))

    def stream_weights(self):
        return [self.w_in, self.w_out]

    def state_need(self):
        return {"S": StateNeed((self.heads, self.dim, self.dim))}

    def _mix(self, ctx, h, app):
        ops, m = ctx.ops, self.inner
        proj = ops.linear(h, self.w_in, None, out_dtype=ctx.dtype)                    # [T, r | k | v | g | a | w1 (| 0)]
        wz = ops.low_rank_out(proj, 5 * m, self.w_w2, self.w0, "tanh")                # float32 [T, heads * dim]
        o = ops.generalized_delta_rule(proj, 0, m, 2 * m, 4 * m, self.b_a, wz, self.decay_coef, app.state["S"], ctx.plan,
                                       self.heads, self.dim, UNIT_EPS)
        return ops.gated_group_norm(o, proj, 3 * m, self.norm_w, self.heads, self.eps, ctx.dtype, gate_first=False,
                                    gate="sigmoid")

    def forward(self, ctx, h, residual, app):
        return ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, residual=residual)

    def branches(self, ctx, h, app):
        import torch
        return [(ctx.ops.linear(self._mix(ctx, h, app), self.w_out, None, out_dtype=torch.float32), 1.0)]


register_part("mixer", "generalized_delta_rule", GeneralizedDeltaRule)
