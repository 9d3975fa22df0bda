"""Vipolix's configuration, read from its own config.json.

The file is nested: `vocab`, `width`, `norm.eps`, optionally `token_side.dim` (the per-layer input taken
from the token ids), and `layers`, a list with one entry per layer: `type` (which mixer the layer has:
`gla` or `parallel`), `mixer` (that mixer's sizes and constants) and `mlp` (the experts', or null for a
layer without a feed-forward).  The architecture is named by a top-level `architecture` string.  Every
size and constant is taken from there (the rank of the decays' two-step products is the stored tensors';
`decay_rank` names it for random-weights mode); what the design knows is checked here, key by key, so that
an error names the key.
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig

MIXERS = ("gla", "parallel")
MLPS = ("moe",)


def _get(d: dict, path: str, kind, where: str, positive: bool = True):
    cur: Any = d
    for key in path.split("."):
        if not isinstance(cur, dict) or key not in cur or cur[key] is None:
            raise ConfigError(f"VipolixConfig: {where}{path} is missing")
        cur = cur[key]
    if isinstance(cur, bool) or not isinstance(cur, (int, float)) or (kind is int and int(cur) != cur):
        raise ConfigError(f"VipolixConfig: {where}{path} = {cur!r}, expected {'a whole number' if kind is int else 'a number'}")
    cur = kind(cur)
    if positive and not cur > 0:
        raise ConfigError(f"VipolixConfig: {where}{path} = {cur} must be positive")
    return cur


@dataclasses.dataclass(frozen=True)
class VipolixConfig(ModelConfig):
    architecture: ClassVar[str] = "Vipolix"

    vocab: int
    width: int
    norm_eps: float
    side_dim: int          # 0: no per-layer input from the token ids
    layers: tuple          # the entries of config.json's `layers`, checked, as plain dicts

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "VipolixConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("VipolixConfig: layers is missing or empty")
        side = d.get("token_side")
        cfg = cls(vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""), norm_eps=_get(d, "norm.eps", float, ""),
                  side_dim=0 if side is None else _get(d, "token_side.dim", int, ""), layers=tuple(copy.deepcopy(layers)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            at = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"VipolixConfig: layers[{i}] is not an object")
            if layer.get("type") not in MIXERS:
                raise ConfigError(f"VipolixConfig: {at}type = {layer.get('type')!r} is not one of {MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"VipolixConfig: {at}mixer is missing")
            if layer["type"] == "gla":
                for key in ("heads", "dim", "vdim"):
                    _get(m, key, int, at + "mixer.")
                _get(m, "tau", float, at + "mixer.")
                if m.get("decay_rank") is not None:
                    _get(m, "decay_rank", int, at + "mixer.")
            else:
                for key in ("left.dim", "left.heads", "left.kv_heads", "left.vdim", "left.conv", "left.mask.size",
                            "left.rot.dims", "right.dim", "right.heads"):
                    _get(m, key, int, at + "mixer.")
                for key in ("left.scale", "left.rot.base"):
                    _get(m, key, float, at + "mixer.")
                _get(m, "left_scale", float, at + "mixer.", positive=False)
                _get(m, "right_scale", float, at + "mixer.", positive=False)
                a = m["left"]
                if a["heads"] % a["kv_heads"]:
                    raise ConfigError(f"VipolixConfig: {at}mixer.left.heads is not a multiple of kv_heads")
                if a["rot"]["dims"] % 2 or a["rot"]["dims"] > a["dim"]:
                    raise ConfigError(f"VipolixConfig: {at}mixer.left.rot.dims = {a['rot']['dims']} is odd or more than dim")
                if m["right"].get("decay_rank") is not None:
                    _get(m, "right.decay_rank", int, at + "mixer.")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLPS:
                    raise ConfigError(f"VipolixConfig: {at}mlp.kind = {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                      f"is not one of {MLPS}")
                _get(mlp, "expert.ff", int, at + "mlp.")
                _get(mlp, "expert.limit", float, at + "mlp.")
                experts = _get(mlp, "router.experts", int, at + "mlp.")
                top = _get(mlp, "router.top", int, at + "mlp.")
                _get(mlp, "router.scale", float, at + "mlp.", positive=False)
                if top > experts:
                    raise ConfigError(f"VipolixConfig: {at}mlp.router.top = {top} is more than its {experts} experts")
                if mlp["router"].get("groups") is not None:
                    count = _get(mlp, "router.groups.count", int, at + "mlp.")
                    keep = _get(mlp, "router.groups.keep", int, at + "mlp.")
                    if experts % count or keep > count or keep * (experts // count) < top:
                        raise ConfigError(f"VipolixConfig: {at}mlp.router.groups = {count} groups, {keep} kept, do not fit "
                                          f"{experts} experts of which {top} are chosen")
                if mlp.get("shared") is not None:
                    _get(mlp, "shared.ff", int, at + "mlp.")
                    _get(mlp, "shared.limit", float, at + "mlp.")

    def check_dtype(self, dtype: str) -> None:
        """Nothing is refused: every part of this design has a kernel for every size in both compute types (rows
        that are no multiples of 16 bytes take the slower ones)."""

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": copy.deepcopy(list(self.layers))}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        return d
