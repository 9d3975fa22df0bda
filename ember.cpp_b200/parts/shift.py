"""Token shift: a mixer reads, in place of its normed input h_t, a blend of it with the row of the token
before: h_t + (h_(t-1) - h_t) * mu, element by element, mu a learned vector of the model width.  The
row before a sequence's first token is zeros; h_(t-1) is the row as it was before any blending.  (The
mixing of neighbouring tokens that the RWKV models put in front of their projections: Peng et al.,
"RWKV: Reinventing RNNs for the Transformer Era".)

It is a mixer that wraps another: it carries the last row of every sequence from step to step (one
`StateNeed` of the model width under the name "shift"), blends, and hands the blended rows to the
mixer inside, whose cache and state needs pass through (its states under "inner.").
"""
from __future__ import annotations

import dataclasses

from .base import Mixer, StateNeed, WeightSpec, build_part, register_part
from .spec import PartSpec


class TokenShift(Mixer):

    def __init__(self, prefix: str, width: int, inner, weight: str = "shift"):
        """inner: the PartSpec (or its (kind, prefix, params)) of the mixer that reads the blended rows; its
        tensor prefix is given whole."""
        super().__init__(prefix)
        self.width = int(width)
        self.weight_name = prefix + weight
        self.inner = build_part("mixer", inner if isinstance(inner, PartSpec) else PartSpec(*inner))
        self.graph_safe = self.inner.graph_safe
        self.mu = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.width,), mean=0.5, std=0.2)] + self.inner.weight_specs()

    def load(self, get, runtime):
        self.mu = runtime.vector(get(self.weight_name))
        self.inner.load(get, runtime)

    def stream_weights(self):
        return self.inner.stream_weights()

    def cache_need(self):
        return self.inner.cache_need()

    def state_need(self):
        need = {"shift": StateNeed((self.width,))}
        s = self.inner.state_need()
        if s is not None:
            for key, one in (s.items() if isinstance(s, dict) else [("", s)]):
                need[f"inner.{key}"] = one
        return need

    def _inside(self, app):
        s = self.inner.state_need()
        if s is None:
            state = None
        elif isinstance(s, dict):
            state = {key: app.state[f"inner.{key}"] for key in s}
        else:
            state = app.state["inner."]
        return dataclasses.replace(app, state=state)

    def _blend(self, ctx, h, app):
        return ctx.ops.token_shift(h, self.mu, app.state["shift"], ctx.plan)

    def forward(self, ctx, h, residual, app):
        return self.inner.forward(ctx, self._blend(ctx, h, app), residual, self._inside(app))

    def branches(self, ctx, h, app):
        return self.inner.branches(ctx, self._blend(ctx, h, app), self._inside(app))


register_part("mixer", "token_shift", TokenShift)
