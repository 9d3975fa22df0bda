"""Interfaces of the parts and their registry.

A part is built from a `PartSpec` alone: its sizes and constants are constructor parameters, its
tensors are named by a prefix that the architecture gives it.  No part knows which model it is in.

Roles and what each must provide:

  norm      forward(ctx, x, out_dtype) -> tensor                     (x: fp32 residual stream)
  mixer     forward(ctx, h, residual, app) -> new residual stream    (h: normed input)
            cache_need() -> CacheNeed | None, state_need() -> StateNeed | {name: StateNeed} | None
  ffn       forward(ctx, h, residual) -> new residual stream
            (mixer and ffn also: branches(ctx, h[, app]) -> [(float32 rows, factor)], the output as a weighted
            sum that the caller adds itself, for arrangements that norm a sublayer's output before the sum;
            a norm's add_normed(ctx, x, branches) makes that sum, norms it and adds it to the stream.  A branch
            may carry a third entry (gain, eps): its rows are then divided by their root mean square and
            multiplied by that gain before they are weighted; `plain_branches` does that for a consumer that has
            no kernel for it)
  embed     forward(ctx, x, state) -> x     (adds to the embedded rows; state_need() as a mixer's: what it
            carries per sequence, kept by the cache beside the layers' states)
  position  embedding_table() -> tensor | None, max_positions() -> int | None,
            apply_qk(ctx, qkv, n_heads, kv_heads, head_dim) (in place; default: nothing)
  addon     forward(ctx, x) -> x            (something added to the stream after a layer's sublayers, reading the
            stream itself and, where it sets `needs_tokens`, the step's token ids)
  block     forward(ctx, x, app) -> x       (the arrangement of the parts above)

Every part lists its tensors with `weight_specs()` (name, stored shape, how random-weights mode
fills it) and receives them in `load(get, runtime)`.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable

from .spec import PartSpec


@dataclasses.dataclass(frozen=True)
class WeightSpec:
    """One tensor of a checkpoint: its full name, its shape as stored, and how the
    random-weights mode draws it: N(mean, std)."""
    name: str
    shape: tuple[int, ...]
    mean: float = 0.0
    std: float = 0.02
    integer: bool = False     # an integer table (kept as int32); none in GPT-2
    below: int = 0            # integer tables in random-weights mode: every row holds distinct values of [0, below)
    free: tuple[int, ...] = ()  # dimensions whose size the checkpoint gives (a rank that no configuration key names);
                                # `shape` holds there the size that random-weights mode draws


@dataclasses.dataclass(frozen=True)
class CacheNeed:
    """What a mixer wants from the cache: all keys (`full`), the last `window` of them (`window`), with
    the first `keep_first` positions of the sequence kept beside the window for good, or the keys of
    the query's own run of `window` positions counted from the sequence's start (`chunk`).  Values may
    have a row size of their own (`value_dim`; 0: the keys')."""
    kind: str                 # "full" | "window" | "chunk"
    kv_heads: int
    head_dim: int
    window: int = 0
    keep_first: int = 0
    value_dim: int = 0

    @property
    def v_dim(self) -> int:
        return self.value_dim or self.head_dim


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size: `shape` values of `dtype` ("float32" or "int32") per
    sequence, set to `init` when a sequence starts.  A mixer that keeps several tensors returns a
    dict of these by name from `state_need()`, and finds a dict of tensors in `app.state`."""
    shape: tuple[int, ...]
    init: float = 0.0
    dtype: str = "float32"


class Part:
    role = ""
    # False for a part whose forward works on the host (reads device values back, loops in Python):
    # an engine with such a part runs every step launch by launch instead of replaying a graph
    graph_safe = True

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def stream_weights(self) -> list:
        """The weight matrices that this part's forward streams through `ops.linear`, in that order
        (as prepared by load()).  A hint for the kernels: a block announces them so that one product's
        launch can ask the next product's weights into L2.  The default names none."""
        return []

    def load(self, get: Callable[[str], Any], runtime) -> None:
        """Fetch the tensors named in weight_specs() with `get(name)` (as stored, on the
        runtime's device) and keep them in the form the kernels want."""


def plain_branches(ctx, branches):
    """`branches` with every pending norm of a branch's own carried out: [(float32 rows, factor)]."""
    import torch
    out = []
    for b in branches:
        if len(b) > 2 and b[2] is not None:
            gain, eps = b[2]
            out.append((ctx.ops.rmsnorm(b[0].contiguous(), gain, eps, torch.float32), b[1]))
        else:
            out.append((b[0], b[1]))
    return out


class Norm(Part):
    role = "norm"

    def forward(self, ctx, x, out_dtype):
        raise NotImplementedError

    def add_normed(self, ctx, x, branches):
        """x + norm(sum of factor * rows over `branches`), the sums in float32.  A norm whose kernel
        does all of it in one launch overrides this."""
        total = None
        for rows, factor in plain_branches(ctx, branches):
            term = rows.float() * factor
            total = term if total is None else total + term
        return x + self.forward(ctx, total.contiguous(), x.dtype)


class Mixer(Part):
    role = "mixer"

    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> "StateNeed | dict[str, StateNeed] | None":
        return None

    def forward(self, ctx, h, residual, app):
        raise NotImplementedError

    def branches(self, ctx, h, app):
        """The mixer's output as [(float32 rows [T, width], factor)]: the caller adds factor * rows.
        The default runs forward() onto a stream of zeros."""
        import torch
        zero = torch.zeros((h.shape[0], self.width), dtype=torch.float32, device=h.device)
        return [(self.forward(ctx, h, zero, app), 1.0)]


class FeedForward(Part):
    role = "ffn"
    # True for a feed-forward that reads the step's token ids (`ctx.plan.tokens`): the model then puts ids that
    # a sampler left on the device into the step's description before the layers run
    needs_tokens = False

    def forward(self, ctx, h, residual):
        raise NotImplementedError

    def branches(self, ctx, h):
        """As Mixer.branches."""
        import torch
        zero = torch.zeros((h.shape[0], self.width), dtype=torch.float32, device=h.device)
        return [(self.forward(ctx, h, zero), 1.0)]


class EmbedPart(Part):
    """Something added to the embedded rows before the first layer (rows of a second table chosen by more
    than the token itself).  It reads the step's tokens (`ctx.plan.tokens`)."""
    role = "embed"
    needs_tokens = True

    def state_need(self) -> "StateNeed | dict[str, StateNeed] | None":
        return None

    def forward(self, ctx, x, state):
        raise NotImplementedError


class StreamAddon(Part):
    """Something a layer adds to the residual stream after its sublayers (a per-layer input taken from the
    token ids, for instance).  It reads the float32 stream and returns the new one."""
    role = "addon"
    needs_tokens = False

    def forward(self, ctx, x):
        raise NotImplementedError


class Position(Part):
    role = "position"

    def embedding_table(self):
        return None

    def max_positions(self) -> int | None:
        return None

    def apply_qk(self, ctx, qkv, n_heads: int, kv_heads: int, head_dim: int) -> None:
        return None


class Block(Part):
    role = "block"

    def __init__(self, norm1: "Norm | None", mixer: Mixer, norm2: "Norm | None", ffn: "FeedForward | None", **more_norms: Norm):
        super().__init__("")
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.more_norms = dict(more_norms)     # the arrangement's further norms, by the names the spec gives them
        self.addons: list = []                 # what the layer adds to the stream after its sublayers (set by the model)

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn, *self.more_norms.values(), *self.addons) if p is not None]

    def add_ons(self, ctx, x):
        for part in self.addons:
            x = part.forward(ctx, x)
        return x

    def forward(self, ctx, x, app):
        raise NotImplementedError


_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {r: {} for r in ("norm", "mixer", "ffn", "position", "block", "embed", "addon")}


def register_part(role: str, kind: str, factory: Callable[..., Part]) -> None:
    """Makes `kind` available to specs for `role`.  `factory(prefix=..., **params)` builds the
    part (for a block: `factory(norm1, mixer, norm2, ffn, **more_norms)`; a norm or a feed-forward
    that the spec leaves out arrives as None)."""
    if role not in _REGISTRY:
        raise ValueError(f"unknown role {role!r}; roles: {sorted(_REGISTRY)}")
    _REGISTRY[role][kind] = factory


def registered(role: str) -> list[str]:
    return sorted(_REGISTRY[role])


def build_part(role: str, spec: PartSpec) -> Part:
    kinds = _REGISTRY[role]
    if spec.kind not in kinds:
        raise ValueError(f"no {role} of kind {spec.kind!r} is registered; registered: {registered(role)}")
    return kinds[spec.kind](prefix=spec.prefix, **spec.params)


def build_block(kind: str, norm1, mixer, norm2, ffn, more_norms=None) -> Block:
    kinds = _REGISTRY["block"]
    if kind not in kinds:
        raise ValueError(f"no block arrangement {kind!r} is registered; registered: {registered('block')}")
    return kinds[kind](norm1, mixer, norm2, ffn, **(more_norms or {}))
