"""Mixers side by side: several mixers read the same normed input and their outputs are added,
each with a fixed factor.

The members are ordinary mixers, given as PartSpecs and built through the registry, so any two
(an attention and a recurrence, two attentions with different windows) can be paired.  At most
one of them may want a cache (a schedule entry has one view of it); their per-sequence states are
kept apart under the member's name.

With `out_norms` every member's output is divided by its root mean square over the model width and
multiplied by a gain of its own before the weighted sum (one tensor name per member, or None for a
member that is added as it is).  The norm travels with the branch (`branches` returns it as the
branch's third entry), so that whoever adds the branches to the stream can norm and add in one launch.
"""
from __future__ import annotations

import dataclasses

from .base import Mixer, WeightSpec, build_part, plain_branches, register_part
from .spec import PartSpec


class ParallelMixers(Mixer):

    def __init__(self, prefix: str, width: int, members, out_norms=None, eps: float = 0.0):
        """members: (name, PartSpec or its (kind, prefix, params), factor) per mixer; a member's tensor
        prefix is given whole (it does not inherit this part's).  out_norms: per member the name (after this
        part's prefix) of the gain that its normed output is multiplied by, or None; eps: inside those norms' roots."""
        super().__init__(prefix)
        self.width, self.eps = int(width), float(eps)
        self.out_norm_names = [None if n is None else prefix + n for n in (out_norms or [None] * len(members))]
        if len(self.out_norm_names) != len(members):
            raise ValueError(f"parallel mixers {prefix!r}: one output norm (or None) for each member")
        self.out_gains = [None] * len(members)
        self.members = []
        for name, spec, factor in members:
            if not isinstance(spec, PartSpec):
                spec = PartSpec(*spec)
            self.members.append((str(name), build_part("mixer", spec), float(factor)))
        if not self.members:
            raise ValueError(f"parallel mixers {prefix!r}: no members")
        if sum(1 for _, m, _ in self.members if m.cache_need() is not None) > 1:
            raise ValueError(f"parallel mixers {prefix!r}: more than one member wants a cache")
        self.graph_safe = all(m.graph_safe for _, m, _ in self.members)

    def weight_specs(self):
        return [w for _, m, _ in self.members for w in m.weight_specs()] + \
            [WeightSpec(n, (self.width,), mean=1.0, std=0.1) for n in self.out_norm_names if n is not None]

    def load(self, get, runtime):
        for _, m, _ in self.members:
            m.load(get, runtime)
        self.out_gains = [None if n is None else runtime.vector(get(n)) for n in self.out_norm_names]

    def stream_weights(self):
        return [w for _, m, _ in self.members for w in m.stream_weights()]

    def cache_need(self):
        for _, m, _ in self.members:
            if m.cache_need() is not None:
                return m.cache_need()
        return None

    def state_need(self):
        need = {}
        for name, m, _ in self.members:
            s = m.state_need()
            if s is None:
                continue
            for key, one in (s.items() if isinstance(s, dict) else [("", s)]):
                need[f"{name}.{key}"] = one
        return need or None

    def _handle(self, app, name, member):
        """The schedule entry as one member sees it: its own state (under its own names), the cache if it wants one."""
        s = member.state_need()
        if s is None:
            state = None
        elif isinstance(s, dict):
            state = {key: app.state[f"{name}.{key}"] for key in s}
        else:
            state = app.state[f"{name}."]
        return dataclasses.replace(app, state=state)

    def branches(self, ctx, h, app):
        runs = [lambda name=name, m=m: m.branches(ctx, h, self._handle(app, name, m)) for name, m, _ in self.members]
        # in a one-token step the members' chains of small kernels can run beside one another (they share their
        # input and nothing else: the cache is one member's, the states are kept apart)
        together = getattr(ctx.ops, "side_by_side", None)
        results = together(runs) if together is not None and ctx.plan.all_single else [run() for run in runs]
        out = []
        for (_, _, factor), rows, gain in zip(self.members, results, self.out_gains):
            if gain is None:
                out += [(b[0], b[1] * factor, *b[2:]) for b in rows]
                continue
            rows = plain_branches(ctx, rows)
            if len(rows) != 1 or rows[0][1] != 1.0:       # the norm is of the member's whole output
                total = sum(r.float() * f for r, f in rows)
                rows = [(total.contiguous(), 1.0)]
            out.append((rows[0][0], factor, (gain, self.eps)))
        return out

    def forward(self, ctx, h, residual, app):
        branches = self.branches(ctx, h, app)
        add = getattr(ctx.ops, "add_branches", None)
        if add is not None and len(branches) <= 8:      # the weighted sum (members' own norms included) and the stream's, one launch
            return add(residual, [(b[0], b[1], b[2][0] if len(b) > 2 and b[2] is not None else None) for b in branches],
                       None, self.eps)
        x = residual
        for rows, f in plain_branches(ctx, branches):
            x = x + f * rows
        return x


register_part("mixer", "parallel", ParallelMixers)
