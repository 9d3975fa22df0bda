"""Vipolix as a ModelSpec.

Token embedding without positions of its own; per layer the `pre_norm` arrangement with RMS norms whose
gains are stored around zero; every mixer reads its input through a token shift (a blend with the row of
the token before, `token_shift`); the mixer inside is gated linear attention, or two members side by
side, added with the configuration's two factors: an attention with biases and short convolutions on q, k
and v, a rotation of a part of every head in neighbouring pairs, a learned factor a head on the scores,
sight limited to the query's own chunk of positions and a sink of score zero; and the generalized delta
rule.  The feed-forward is a set of routed experts of the clamped gated form, with groups, a correction
on the choice and a gated shared expert, or absent; after it a per-layer input taken from the token ids
(`token_side_input`).  A last norm and an untied head.

The design's fixed numbers stand here (1.702 and the + 1 of the clamped gate, the sink's score 0, the
decay's coefficient exp(-1/2)) or in the parts (1e-6 inside the unit keys' root, 1e-20 under the experts'
weights); everything else comes from the configuration.
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.vipolix import VipolixConfig
from ..parts.spec import Application, LayerSpec, ModelSpec, PartSpec

GATE_ALPHA = 1.702
UP_SHIFT = 1.0
SINK_SCORE = 0.0
DECAY_COEF = math.exp(-0.5)


def build_spec(cfg: VipolixConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", name, {"width": d, "eps": eps, "weight": "", "offset": 1.0})  # noqa: E731
    layers, ignored = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "gla":
            more = {"rank": m["decay_rank"]} if m.get("decay_rank") else {}
            inner = PartSpec("gated_linear_attention", p + "mix.", {
                "width": d, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "tau": m["tau"], "eps": eps, **more})
        else:
            a, r = m["left"], m["right"]
            left = PartSpec("causal_attention", p + "mix.left.", {
                "width": d, "n_heads": a["heads"], "kv_heads": a["kv_heads"], "head_dim": a["dim"], "value_dim": a["vdim"],
                "scale": a["scale"], "qkv": ("q", "k", "v"), "out": "o", "stored": "out_in", "bias": False, "suffix": "",
                "qkv_bias": ".b", "conv": (a["conv"], ".conv"), "rotary": (a["rot"]["dims"], a["rot"]["base"], True),
                "head_scale": "temp", "chunk": a["mask"]["size"], "fixed_sink": SINK_SCORE})
            more = {"rank": r["decay_rank"]} if r.get("decay_rank") else {}
            right = PartSpec("generalized_delta_rule", p + "mix.right.", {
                "width": d, "heads": r["heads"], "dim": r["dim"], "eps": eps, "decay_coef": DECAY_COEF, **more})
            inner = PartSpec("parallel", p + "mix.", {"width": d, "members": (
                ("left", left, m["left_scale"]), ("right", right, m["right_scale"]))})
        mixer = PartSpec("token_shift", p, {"width": d, "inner": inner})
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None:
            router, shared = mlp["router"], mlp.get("shared")
            groups = router.get("groups") or {"count": 1, "keep": 1}
            ffn = PartSpec("routed_experts", p + "mlp.", {
                "width": d, "experts": router["experts"], "top": router["top"], "inner": mlp["expert"]["ff"],
                "route_scale": router["scale"], "groups": groups["count"], "keep_groups": groups["keep"],
                "limit": mlp["expert"]["limit"], "alpha": GATE_ALPHA, "shift": UP_SHIFT,
                "shared_inner": shared["ff"] if shared else 0, "shared_limit": shared["limit"] if shared else 0.0,
                "shared_gate": "sg" if shared else None})
        else:
            ignored.append(rf"l{i}\.norm2")
        addons = ()
        if cfg.side_dim:
            addons = (PartSpec("token_side_input", p, {"width": d, "vocab": cfg.vocab, "dim": cfg.side_dim, "layer": i,
                                                       "layers": len(cfg.layers), "eps": eps}),)
        layers.append(LayerSpec("pre_norm", norm(p + "norm1"), mixer, norm(p + "norm2") if ffn is not None else None, ffn,
                                addons=addons))
    return ModelSpec(width=d, vocab_size=cfg.vocab, token_table="embed", position=PartSpec("none", ""),
                     layers=tuple(layers), schedule=tuple(Application(i) for i in range(len(layers))),
                     final_norm=norm("final.norm"), head="head", ignored_tensors=tuple(ignored))


register_architecture(VipolixConfig.architecture, VipolixConfig, build_spec)
