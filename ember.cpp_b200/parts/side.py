"""A per-layer input taken from the token ids, added to the stream after a layer's sublayers.

One table of the whole model holds, for every token id, `dim` values for each layer (layer i reads the
columns [i * dim, (i + 1) * dim)).  With e that slice of the token's row and x the stream:

    g = gelu_tanh(W_gate x) * e        y = W_proj g        x <- x + y / sqrt(mean(y^2) + eps) * w

(the per-layer embeddings of Gemma 3n, reduced to one gate and one projection).  All of it is float32
arithmetic in one launch; the two matrices and the table are read in the compute type.
"""
from __future__ import annotations

from .base import StreamAddon, WeightSpec, register_part


class TokenSideInput(StreamAddon):
    needs_tokens = True

    def __init__(self, prefix: str, width: int, vocab: int, dim: int, layer: int, layers: int, eps: float,
                 table: str = "side.embed", gate: str = "side.gate", proj: str = "side.proj", norm: str = "side.norm",
                 init_std: float = 0.02):
        """table: the whole model's table (its name is given whole, not after `prefix`)."""
        super().__init__(prefix)
        self.width, self.vocab, self.dim, self.layer, self.layers = int(width), int(vocab), int(dim), int(layer), int(layers)
        if not 1 <= self.dim <= 1024 or not 0 <= self.layer < self.layers:
            raise ValueError(f"token side input {prefix!r}: {self.dim} values for layer {self.layer} of {self.layers}")
        self.eps, self.init_std = float(eps), init_std
        self.table_name = table
        self.gate_name, self.proj_name, self.norm_name = prefix + gate, prefix + proj, prefix + norm
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.table_name, (self.vocab, self.layers * self.dim), std=1.0),
                WeightSpec(self.gate_name, (self.dim, self.width), std=self.init_std),
                WeightSpec(self.proj_name, (self.width, self.dim), std=self.init_std),
                WeightSpec(self.norm_name, (self.width,), mean=0.0, std=0.1)]

    def load(self, get, runtime):
        self.table = runtime.table(get(self.table_name))
        self.w_gate = runtime.matrix(get(self.gate_name))
        self.w_proj = runtime.matrix(get(self.proj_name))
        self.w_norm = runtime.vector(get(self.norm_name))

    def forward(self, ctx, x):
        return ctx.ops.side_input(x, ctx.plan, self.table, self.layer * self.dim, self.dim, self.w_gate, self.w_proj,
                                  self.w_norm, self.eps)


register_part("addon", "token_side_input", TokenSideInput)
