"""Sosutar's configuration, read from its own config.json.

The file is nested: `vocab`, `width`, `max_positions`, `norm.eps`, `embedding.scale`, `logit_scale`, and
`layers`, a list with one entry per layer: `type` (which mixer the layer has: `mlstm` or `parallel`),
`mixer` (that mixer's sizes and constants), `mlp` (the feed-forward's, or null for a layer without
one) and optionally `weights_of`, the index of the layer whose tensors this layer runs with (it
then has none of its own, and the rest of its entry equals that layer's).  The architecture is named
by a top-level `architecture` string.  Every size and constant is taken from there; what the design
knows is checked here, key by key, so that an error names the key.
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig

MIXERS = ("mlstm", "parallel")
MLPS = ("dense",)


def _get(d: dict, path: str, kind, where: str, positive: bool = True):
    cur: Any = d
    for key in path.split("."):
        if not isinstance(cur, dict) or key not in cur or cur[key] is None:
            raise ConfigError(f"SosutarConfig: {where}{path} is missing")
        cur = cur[key]
    if isinstance(cur, bool) or not isinstance(cur, (int, float)) or (kind is int and int(cur) != cur):
        raise ConfigError(f"SosutarConfig: {where}{path} = {cur!r}, expected {'a whole number' if kind is int else 'a number'}")
    cur = kind(cur)
    if positive and not cur > 0:
        raise ConfigError(f"SosutarConfig: {where}{path} = {cur} must be positive")
    return cur


@dataclasses.dataclass(frozen=True)
class SosutarConfig(ModelConfig):
    architecture: ClassVar[str] = "Sosutar"

    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple          # the entries of config.json's `layers`, checked, as plain dicts

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "SosutarConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("SosutarConfig: layers is missing or empty")
        cfg = cls(vocab=_get(d, "vocab", int, ""), width=_get(d, "width", int, ""),
                  max_positions=_get(d, "max_positions", int, ""), norm_eps=_get(d, "norm.eps", float, ""),
                  embedding_scale=_get(d, "embedding.scale", float, "", positive=False),
                  logit_scale=_get(d, "logit_scale", float, "", positive=False), layers=tuple(copy.deepcopy(layers)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            at = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"SosutarConfig: layers[{i}] is not an object")
            if layer.get("type") not in MIXERS:
                raise ConfigError(f"SosutarConfig: {at}type = {layer.get('type')!r} is not one of {MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"SosutarConfig: {at}mixer is missing")
            if layer["type"] == "mlstm":
                for key in ("heads", "dim", "vdim"):
                    _get(m, key, int, at + "mixer.")
                _get(m, "gate_cap", float, at + "mixer.")
            else:
                for key in ("left.dim", "left.heads", "left.kv_heads", "left.vdim", "left.mask.size", "left.q_temp.every",
                            "right.width"):
                    _get(m, key, int, at + "mixer.")
                _get(m, "left.scale", float, at + "mixer.")
                _get(m, "left.q_temp.coef", float, at + "mixer.", positive=False)
                if m["left"]["heads"] % m["left"]["kv_heads"]:
                    raise ConfigError(f"SosutarConfig: {at}mixer.left.heads is not a multiple of kv_heads")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLPS:
                    raise ConfigError(f"SosutarConfig: {at}mlp.kind = {mlp.get('kind') if isinstance(mlp, dict) else mlp!r} "
                                      f"is not one of {MLPS}")
                _get(mlp, "ff", int, at + "mlp.")
            src = layer.get("weights_of")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(self.layers) or src == i:
                    raise ConfigError(f"SosutarConfig: {at}weights_of = {src!r} must name another layer")
                owner = self.owner_of(i)
                if owner is None:
                    raise ConfigError(f"SosutarConfig: {at}weights_of = {src} leads to no layer with tensors of its own")
                if self.layers[owner].get("type") != layer["type"]:
                    raise ConfigError(f"SosutarConfig: {at}weights_of = {src} names a layer of another type")

    def owner_of(self, i: int):
        """The layer whose tensors layer i runs with: itself, or where its `weights_of` leads (a layer named there may
        name another in turn); None if that ends nowhere."""
        seen = set()
        while isinstance(self.layers[i], dict) and self.layers[i].get("weights_of") is not None:
            seen.add(i)
            i = self.layers[i]["weights_of"]
            if isinstance(i, bool) or not isinstance(i, int) or not 0 <= i < len(self.layers) or i in seen:
                return None
        return i

    def check_dtype(self, dtype: str) -> None:
        """Nothing is refused: every part of this design has a kernel for every size in both compute types (rows
        that are no multiples of 16 bytes take the slower ones)."""

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
                "layers": copy.deepcopy(list(self.layers))}
