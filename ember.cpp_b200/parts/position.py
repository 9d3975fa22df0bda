"""Position encodings.

GPT-2 adds a learned row per absolute position to the token embedding:
`x[t,:] += wpe[P+t,:]`, and a position past the table is an error (graph_ir.cpp:2410-2420;
kernel graph_ir_cuda.cu:26-32).  The table bounds the context.  `none` is the encoding of a model
whose mixers carry position themselves.

`rotary` rotates pairs of dimensions of a head by an angle that grows with the position: of the
first `dims` dimensions of a vector, dimension i is paired with dimension i + dims/2 and the pair
(u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * f_i,
f_i = base^(-2i/dims); dimensions past `dims` pass unchanged.  With `scaling` (YaRN: Peng, Quesnelle,
Fan, Shippole, "YaRN: Efficient Context Window Extension of Large Language Models") the frequency
of pair i is a blend of f_i / factor and f_i by a ramp over the pair index, the ramp's ends being
the indices whose wavelengths make `fast` and `slow` turns within the `original` context, and both
cos and sin are multiplied by 0.1 ln(factor) + 1.  Frequencies are computed once on the host, the
angles and their cos and sin in float32 on the device.  With `interleaved` the pairs are neighbours:
dimension 2i with dimension 2i + 1.  A mixer that rotates only a part of its heads, or with constants
of its own, builds one of these for itself and calls `rotate`.
"""
from __future__ import annotations

from .base import Position, WeightSpec, register_part


class LearnedAbsolute(Position):

    def __init__(self, prefix: str, width: int, n_positions: int, table: str = "weight", init_std: float = 0.02):
        super().__init__(prefix)
        self.width, self.n_positions = int(width), int(n_positions)
        self.table_name = prefix + table
        self.init_std = init_std
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.table_name, (self.n_positions, self.width), std=self.init_std)]

    def load(self, get, runtime):
        self.table = runtime.table(get(self.table_name))

    def embedding_table(self):
        return self.table

    def max_positions(self):
        return self.n_positions


class NoPosition(Position):

    def __init__(self, prefix: str = ""):
        super().__init__(prefix)


class Rotary(Position):

    def __init__(self, prefix: str = "", dims: int = 0, base: float = 10000.0, scaling: dict | None = None,
                 interleaved: bool = False):
        super().__init__(prefix)
        import math
        self.dims, self.base, self.interleaved = int(dims), float(base), bool(interleaved)
        if self.dims <= 0 or self.dims % 2:
            raise ValueError(f"rotary {prefix!r}: {self.dims} rotated dimensions (an even number)")
        half = self.dims // 2
        freqs = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        self.magnitude = 1.0
        if scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])

            def pair_at(turns):      # the pair index whose wavelength makes `turns` turns within the original context
                return self.dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(self.base))
            lo = max(math.floor(pair_at(float(scaling["fast"]))), 0)
            hi = min(math.ceil(pair_at(float(scaling["slow"]))), self.dims - 1)
            for i in range(half):
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                freqs[i] = freqs[i] / factor * ramp + freqs[i] * (1.0 - ramp)
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.freqs_host = freqs
        self.freqs = None

    def load(self, get, runtime):
        import torch
        self.freqs = torch.tensor(self.freqs_host, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def rotate(self, ctx, src, dst, heads: int, src_col: int, src_head: int, dst_col: int, dst_head: int, width: int):
        """dst[t, dst_col + h * dst_head + (0..width)] = the rotated src[t, src_col + h * src_head + (0..width)] for
        h < heads, by each token's position; src and dst may be one tensor (in place)."""
        return ctx.ops.rotate(src, dst, ctx.plan.positions, heads, src_col, src_head, dst_col, dst_head, width,
                              self.freqs, self.magnitude, self.dims, **({"interleaved": True} if self.interleaved else {}))

    def apply_qk(self, ctx, qkv, n_heads: int, kv_heads: int, head_dim: int) -> None:
        self.rotate(ctx, qkv, qkv, n_heads + kv_heads, 0, head_dim, 0, head_dim, head_dim)


register_part("position", "rotary", Rotary)
register_part("position", "learned_absolute", LearnedAbsolute)
register_part("position", "none", NoPosition)
