"""Causal multi-head attention over the cache, with a fused q|k|v projection.

ember.cpp's GPT-2 block: `qkv = h W^T + b`, split into q | k | v by columns
(sizes [H*hd, KV*hd, KV*hd], graph_ir.cpp:733-735), write k and v at their positions, then for
each query the scaled scores over the keys up to its own position, softmax, weighted sum of the
values (graph_ir.cpp:2539-2620; cpu_attention.cpp:92-211), and the output projection whose result
is added to the residual stream (graph_ir.cpp:742, 754).  Query head h reads key/value head
h // (H / KV) (cpu_attention.cpp:127).  With `window` > 0 a query at position p sees positions
p-window+1 .. p (cpu_attention.cpp, swa_visible_ranges).  The scale is a parameter: the
architecture computes it (GPT-2: 1/sqrt(hd), optionally divided by layer+1).

Beyond GPT-2's shape, all as parameters: the first `keep_first` positions of a sequence stay
visible beside the window (query p sees key j <= p if p - j < window or j < keep_first; the cache
keeps their pages); values may have a row size of their own (`value_dim`); q, k and v may be
stored as three matrices (`qkv` a tuple of three names: they are laid end to end at load, so the
step still makes one product); tensor names may carry no `.weight` suffix (`suffix`).

Further options, each off by default and each a parameter (`parts/attention.py::CausalAttention`):
`qk_norm` = (name of q's gain, name of k's gain): q and k are each divided by their root mean square over
the whole projection, before they are cut into heads, and multiplied by a gain of that size; `value_norm`:
every value head is divided by its own root mean square before it is cached; `q_temp` = (coef, every): q at
position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1); `distance_slope_base` = b: the score of
key j for query i of head h loses 2^(-b (h + 1) / heads) * (i - j); `sink`: the name of one learned number per
head whose exponential is added to the softmax's denominator (it has no key and no value); `gate`: the name of a
matrix W_g, the heads laid end to end are multiplied by sigmoid(W_g h) before the output projection.  With a norm
on q or k or v, or a gate, the projection q | k | v (| g) is left in float32 (the norms read it unrounded) and
the normed rows are rounded to the compute type once.

And, again each a parameter: `qkv_bias` = suffix: q, k and v (stored as three matrices) have biases of that
suffix, added in the projection, and the output projection has none; `conv` = (taps, suffix): a short causal
convolution over time on every channel of q, k and v (a filter [channels, taps] a tensor, the last tap on the
current token, zeros before the sequence's start, no bias, no activation) directly after the projection; the
last taps - 1 projected rows of a sequence are its state ("conv"); `rotary` = (dims, base, interleaved): the
mixer rotates the first `dims` dimensions of every q and k head itself, neighbours (2i, 2i + 1) paired where
`interleaved`; `head_scale`: the name of one learned factor a query head on its scores; `chunk` = size: query i
sees key j <= i only if floor(i / size) = floor(j / size), counted from the sequence's position 0 (the cache
then keeps the pages of the query's own run alone); `fixed_sink` = s: a sink whose score is the constant s.
"""
from __future__ import annotations

from .base import CacheNeed, Mixer, StateNeed, WeightSpec, register_part


def slope_base_or_sink(slope_base, sink) -> bool:
    return slope_base is not None or sink is not None


class CausalAttention(Mixer):

    def __init__(self, prefix: str, width: int, n_heads: int, kv_heads: int, head_dim: int, scale: float,
                 window: int = 0, qkv="c_attn", out: str = "c_proj", stored: str = "in_out",
                 bias: bool = True, init_std: float = 0.02, out_init_std: float = 0.02, bias_init_std: float = 0.01,
                 keep_first: int = 0, value_dim: int | None = None, suffix: str = ".weight", qk_norm=None,
                 value_norm: bool = False, norm_eps: float = 0.0, q_temp=None, distance_slope_base: float | None = None,
                 sink: str | None = None, gate: str | None = None, qkv_bias: str | None = None, conv=None, rotary=None,
                 head_scale: str | None = None, chunk: int = 0, fixed_sink: float | None = None):
        super().__init__(prefix)
        if n_heads % kv_heads:
            raise ValueError(f"attention {prefix!r}: {n_heads} heads are not a multiple of {kv_heads} key/value heads")
        if not 1 <= head_dim <= 256:
            raise ValueError(f"attention {prefix!r}: head size {head_dim} is not in [1, 256]")
        if stored not in ("in_out", "out_in"):
            raise ValueError(f"attention {prefix!r}: stored = {stored!r}")
        self.width, self.n_heads, self.kv_heads, self.head_dim = int(width), int(n_heads), int(kv_heads), int(head_dim)
        self.scale, self.window, self.keep_first = float(scale), int(window), int(keep_first)
        # keep_first or an explicit value size take the kernels that know both (and every head size, also in bfloat16)
        self.qk_norm_names = None if qk_norm is None else tuple(prefix + n for n in qk_norm)
        self.value_norm, self.norm_eps = bool(value_norm), float(norm_eps)
        self.q_temp = None if q_temp is None else (float(q_temp[0]), int(q_temp[1]))
        if self.q_temp is not None and self.q_temp[1] <= 0:
            raise ValueError(f"attention {prefix!r}: a temperature that grows every {self.q_temp[1]} positions")
        self.slope_base = None if distance_slope_base is None else float(distance_slope_base)
        self.sink_name = None if sink is None else prefix + sink
        self.gate_name = None if gate is None else prefix + gate
        # rows that pass a norm, a temperature or a gate between the projection and the attention
        self.prepared = self.qk_norm_names is not None or self.value_norm or self.q_temp is not None or self.gate_name is not None
        self.fixed_sink = None if fixed_sink is None else float(fixed_sink)
        self.chunk = int(chunk)
        self.head_scale_name = None if head_scale is None else prefix + head_scale
        self.conv = None if conv is None else (int(conv[0]), str(conv[1]))
        self.qkv_bias_suffix = qkv_bias
        self.rotary = None
        if rotary is not None:
            from .position import Rotary
            self.rotary = Rotary(prefix, dims=int(rotary[0]), base=float(rotary[1]), interleaved=bool(rotary[2]))
            if self.rotary.dims > head_dim:
                raise ValueError(f"attention {prefix!r}: {self.rotary.dims} rotated dimensions of a head of {head_dim}")
        if self.chunk < 0 or (self.chunk and window):
            raise ValueError(f"attention {prefix!r}: chunk {self.chunk} (not negative, and not beside a window)")
        if self.fixed_sink is not None and sink is not None:
            raise ValueError(f"attention {prefix!r}: a learned sink or a fixed one")
        if self.conv is not None and not 1 <= self.conv[0] <= 16:
            raise ValueError(f"attention {prefix!r}: a convolution of {self.conv[0]} taps is not in [1, 16]")
        if (qkv_bias is not None or self.conv is not None) and (isinstance(qkv, str) or bias):
            raise ValueError(f"attention {prefix!r}: biases on q, k and v alone and convolutions come with q, k and v "
                             "stored as three matrices, without the fused projection's biases")
        self.biased = (self.slope_base is not None or self.sink_name is not None or self.fixed_sink is not None
                       or self.chunk > 0 or self.head_scale_name is not None)
        if (self.prepared or slope_base_or_sink(distance_slope_base, sink)) and bias:
            raise ValueError(f"attention {prefix!r}: norms, gates, slopes and sinks come without biases")
        self.extended = int(keep_first) > 0 or value_dim is not None or self.prepared or self.biased
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        if not 1 <= self.value_dim <= 256:
            raise ValueError(f"attention {prefix!r}: value size {self.value_dim} is not in [1, 256]")
        if self.keep_first < 0 or self.window < 0:
            raise ValueError(f"attention {prefix!r}: window {self.window}, keep_first {self.keep_first}")
        self.split = not isinstance(qkv, str)      # q, k and v stored as three matrices
        if self.split and (len(qkv) != 3 or bias):
            raise ValueError(f"attention {prefix!r}: three names for q, k and v, and no biases with them")
        self.qkv_name = tuple(prefix + n for n in qkv) if self.split else prefix + qkv
        self.out_name, self.stored, self.bias, self.suffix = prefix + out, stored, bias, suffix
        self.init_std, self.out_init_std, self.bias_init_std = init_std, out_init_std, bias_init_std
        self.q_width = self.n_heads * self.head_dim
        self.o_width = self.n_heads * self.value_dim
        self.widths = (self.q_width, self.kv_heads * self.head_dim, self.kv_heads * self.value_dim)
        self.qkv_width = sum(self.widths)
        self.w_qkv = self.b_qkv = self.w_out = self.b_out = None
        self.q_gain = self.k_gain = self.sinks = self.slopes = None

    def _shape(self, n_in, n_out):
        return (n_in, n_out) if self.stored == "in_out" else (n_out, n_in)

    def weight_specs(self):
        if self.split:
            specs = [WeightSpec(n + self.suffix, self._shape(self.width, w), std=self.init_std)
                     for n, w in zip(self.qkv_name, self.widths)]
        else:
            specs = [WeightSpec(self.qkv_name + self.suffix, self._shape(self.width, self.qkv_width), std=self.init_std)]
        specs.append(WeightSpec(self.out_name + self.suffix, self._shape(self.o_width, self.width), std=self.out_init_std))
        if self.bias:
            specs += [WeightSpec(self.qkv_name + ".bias", (self.qkv_width,), std=self.bias_init_std),
                      WeightSpec(self.out_name + ".bias", (self.width,), std=self.bias_init_std)]
        if self.qk_norm_names is not None:
            specs += [WeightSpec(self.qk_norm_names[0], (self.q_width,), mean=1.0, std=0.1),
                      WeightSpec(self.qk_norm_names[1], (self.widths[1],), mean=1.0, std=0.1)]
        if self.sink_name is not None:
            specs.append(WeightSpec(self.sink_name, (self.n_heads,), std=1.0))
        if self.gate_name is not None:
            specs.append(WeightSpec(self.gate_name + self.suffix, self._shape(self.width, self.o_width), std=self.init_std))
        if self.qkv_bias_suffix is not None:
            specs += [WeightSpec(n + self.qkv_bias_suffix, (w,), std=self.bias_init_std * 10) for n, w in zip(self.qkv_name, self.widths)]
        if self.conv is not None:
            specs += [WeightSpec(n + self.conv[1], (w, self.conv[0]), std=0.5) for n, w in zip(self.qkv_name, self.widths)]
        if self.head_scale_name is not None:
            specs.append(WeightSpec(self.head_scale_name, (self.n_heads,), mean=1.0, std=0.2))
        return specs

    def load(self, get, runtime):
        import torch
        if runtime.dtype == torch.bfloat16 and not self.extended and (self.head_dim % 16 or self.width % 8):
            # (the true 32-bit path takes every head size up to 256 and every width)
            raise ValueError(f"attention {self.prefix!r}: the bfloat16 kernels take head sizes that are multiples of 16 "
                             f"and widths that are multiples of 8 (here {self.head_dim} and {self.width}); "
                             "the float32 path takes this model")
        t = self.stored == "in_out"
        if self.split:
            self.w_qkv = torch.cat([runtime.matrix(get(n + self.suffix), transpose=t) for n in self.qkv_name]).contiguous()
        else:
            self.w_qkv = runtime.matrix(get(self.qkv_name + self.suffix), transpose=t)
        self.w_out = runtime.matrix(get(self.out_name + self.suffix), transpose=t)
        if self.gate_name is not None:      # the gate's rows under q | k | v, each part from a multiple of 8 columns on
            self.gate_col = -(-self.qkv_width // 8) * 8
            pad = torch.zeros((self.gate_col - self.qkv_width, self.width), dtype=self.w_qkv.dtype, device=self.w_qkv.device)
            self.w_qkv = torch.cat([self.w_qkv, pad, runtime.matrix(get(self.gate_name + self.suffix), transpose=t)]).contiguous()
        if self.qk_norm_names is not None:
            self.q_gain, self.k_gain = (runtime.vector(get(n)) for n in self.qk_norm_names)
        if self.sink_name is not None:
            self.sinks = runtime.vector(get(self.sink_name))
        if self.slope_base is not None:
            self.slopes = torch.tensor([2.0 ** (-self.slope_base * (h + 1) / self.n_heads) for h in range(self.n_heads)],
                                       dtype=torch.float32, device=self.w_qkv.device)
        if self.bias:
            self.b_qkv = runtime.vector(get(self.qkv_name + ".bias"))
            self.b_out = runtime.vector(get(self.out_name + ".bias"))
        if self.qkv_bias_suffix is not None:
            self.b_qkv = torch.cat([runtime.vector(get(n + self.qkv_bias_suffix)) for n in self.qkv_name]).contiguous()
        if self.conv is not None:
            self.conv_w = torch.cat([runtime.vector(get(n + self.conv[1])) for n in self.qkv_name]).contiguous()
            self.conv_b = torch.zeros(self.qkv_width, dtype=torch.float32, device=self.conv_w.device)
        if self.rotary is not None:
            self.rotary.load(get, runtime)
        if self.fixed_sink is not None:
            self.sinks = torch.full((self.n_heads,), self.fixed_sink, dtype=torch.float32, device=self.w_qkv.device)
        self.head_scales = None
        if self.head_scale_name is not None:
            self.head_scales = runtime.vector(get(self.head_scale_name))
            # (the tensor-core kernels take their exponents against a running maximum of the raw products, which
            # needs factors above zero; any other head takes the plain kernel)
            self.head_scales_positive = bool((self.head_scales > 0).all())

    def stream_weights(self):
        return [self.w_qkv, self.w_out]

    def state_need(self):
        if self.conv is None or self.conv[0] <= 1:
            return None
        return {"conv": StateNeed((self.conv[0] - 1, self.qkv_width))}     # the projected rows before the step's first, oldest first

    def cache_need(self):
        if self.chunk > 0:
            return CacheNeed("chunk", self.kv_heads, self.head_dim, self.chunk, 0,
                             0 if self.value_dim == self.head_dim else self.value_dim)
        windowed = self.window > 0
        return CacheNeed("window" if windowed else "full", self.kv_heads, self.head_dim, self.window,
                         self.keep_first if windowed else 0, 0 if self.value_dim == self.head_dim else self.value_dim)

    def _attend(self, ctx, h, app):
        ops = ctx.ops
        if self.prepared:
            import torch
            proj = ops.linear(h, self.w_qkv, None, out_dtype=torch.float32)          # float32 [T, q | k | v (| 0 | g)]
            coef, every = self.q_temp or (0.0, 1)
            qkv = ops.qkv_norm(proj, ctx.plan.positions, self.n_heads, self.kv_heads, self.head_dim, self.value_dim, ctx.dtype,
                               q_gain=self.q_gain, k_gain=self.k_gain, unit_values=self.value_norm, eps=self.norm_eps,
                               temp_coef=coef, temp_every=every)
            ctx.position.apply_qk(ctx, qkv, self.n_heads, self.kv_heads, self.head_dim)
            o = ops.attention(qkv, app.cache, ctx.plan, self.n_heads, self.kv_heads, self.head_dim, self.scale, self.window,
                              out_dtype=ctx.dtype, store=app.writes_cache, keep_first=self.keep_first if self.window > 0 else 0,
                              value_dim=self.value_dim, slopes=self.slopes, sinks=self.sinks)
            return o if self.gate_name is None else ops.gate_mul(o, proj, self.gate_col, "sigmoid")
        qkv = ops.linear(h, self.w_qkv, self.b_qkv, out_dtype=ctx.dtype)
        if self.conv is not None:
            state = app.state.get("conv") if isinstance(app.state, dict) else None
            qkv = ops.conv_silu(qkv, 0, self.qkv_width, self.conv_w, self.conv_b, state, ctx.plan, act="none")
        ctx.position.apply_qk(ctx, qkv, self.n_heads, self.kv_heads, self.head_dim)
        if self.rotary is not None:
            self.rotary.apply_qk(ctx, qkv, self.n_heads, self.kv_heads, self.head_dim)
        if self.chunk > 0 or self.head_scales is not None:
            return ops.attention(qkv, app.cache, ctx.plan, self.n_heads, self.kv_heads, self.head_dim, self.scale,
                                 self.window, out_dtype=ctx.dtype, store=app.writes_cache, keep_first=0, value_dim=self.value_dim,
                                 slopes=self.slopes, sinks=self.sinks, chunk=self.chunk, head_scales=self.head_scales,
                                 head_scales_positive=self.head_scales is None or self.head_scales_positive)
        if not self.extended:
            return ops.attention(qkv, app.cache, ctx.plan, self.n_heads, self.kv_heads, self.head_dim, self.scale,
                                 self.window, out_dtype=ctx.dtype, store=app.writes_cache)
        return ops.attention(qkv, app.cache, ctx.plan, self.n_heads, self.kv_heads, self.head_dim, self.scale,
                             self.window, out_dtype=ctx.dtype, store=app.writes_cache,
                             keep_first=self.keep_first if self.window > 0 else 0, value_dim=self.value_dim,
                             slopes=self.slopes, sinks=self.sinks)

    def forward(self, ctx, h, residual, app):
        return ctx.ops.linear(self._attend(ctx, h, app), self.w_out, self.b_out, residual=residual)

    def branches(self, ctx, h, app):
        import torch
        return [(ctx.ops.linear(self._attend(ctx, h, app), self.w_out, self.b_out, out_dtype=torch.float32), 1.0)]


register_part("mixer", "causal_attention", CausalAttention)
