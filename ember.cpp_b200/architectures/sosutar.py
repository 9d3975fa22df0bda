"""Sosutar as a ModelSpec.

Token rows times a factor plus a learned row per position (the factor on the token's row alone);
per layer the `sandwich` arrangement with an RMS norm before each sublayer and, in the place of the norm
after it, a gain per channel (`layer_scale`): `x + ls1 * mixer(norm1(x))`, then `x + ls2 * ff(norm2(x))`.
A layer's mixer is the mLSTM (such layers have no feed-forward in the models seen so far, but any layer
may have one or none), or two members side by side on the same input: an attention with a sliding window,
norms on q, k and v, a query temperature, a distance penalty with slopes 2^(-8 (h + 1) / heads), a sink
and a sigmoid output gate, and a minGRU; each member's output is RMS-normed with a gain of its own and the
two are added with a half each.  Feed-forwards are dense with a squared relu.  A layer with `weights_of`
is an entry of the run order that names the other layer's parts: it gets a cache and state of its own.
A last norm, an untied head, and a factor on the logits.

The design's fixed numbers (the slopes' base 8, the half and half of the two members) stand here; everything
else comes from the configuration.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.sosutar import SosutarConfig
from ..parts.spec import Application, LayerSpec, ModelSpec, PartSpec

SLOPE_BASE = 8.0
MEMBER_FACTOR = 0.5


def build_spec(cfg: SosutarConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    norm = lambda name: PartSpec("rmsnorm", name, {"width": d, "eps": eps, "weight": ""})  # noqa: E731
    gain = lambda name: PartSpec("layer_scale", name, {"width": d, "weight": "", "eps": eps})  # noqa: E731
    layers, index_of, schedule = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.get("weights_of") is not None:
            schedule.append(None)       # (filled in below: the owner may come later in the list)
            continue
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "mlstm":
            mixer = PartSpec("mlstm", p + "mix.", {"width": d, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                                                   "gate_cap": m["gate_cap"], "eps": eps})
        else:
            a, r = m["left"], m["right"]
            left = PartSpec("causal_attention", p + "mix.left.", {
                "width": d, "n_heads": a["heads"], "kv_heads": a["kv_heads"], "head_dim": a["dim"], "value_dim": a["vdim"],
                "scale": a["scale"], "window": a["mask"]["size"], "qkv": ("q", "k", "v"), "out": "o", "stored": "out_in",
                "bias": False, "suffix": "", "qk_norm": ("q.norm", "k.norm"), "value_norm": True, "norm_eps": eps,
                "q_temp": (a["q_temp"]["coef"], a["q_temp"]["every"]), "distance_slope_base": SLOPE_BASE, "sink": "sink",
                "gate": "g"})
            right = PartSpec("mingru", p + "mix.right.", {"width": d, "inner": r["width"]})
            mixer = PartSpec("parallel", p + "mix.", {
                "width": d, "members": (("left", left, MEMBER_FACTOR), ("right", right, MEMBER_FACTOR)),
                "out_norms": ("left.out", "right.out"), "eps": eps})
        mlp = layer.get("mlp")
        ffn = None if mlp is None else PartSpec("dense", p + "mlp.", {
            "width": d, "inner": mlp["ff"], "activation": "relu2", "up": "up", "down": "down", "stored": "out_in",
            "bias": False, "suffix": "", "any_size": True})
        more = (("after_mixer", gain(p + "ls1")),) + ((("after_ffn", gain(p + "ls2")),) if ffn is not None else ())
        index_of[i] = len(layers)
        layers.append(LayerSpec("sandwich", norm(p + "norm1"), mixer, norm(p + "norm2") if ffn is not None else None, ffn, more))
        schedule.append(Application(index_of[i]))
    # a layer may run with the tensors of a layer that comes after it in the list, or of one that names a third
    for i in range(len(cfg.layers)):
        if schedule[i] is None:
            schedule[i] = Application(index_of[cfg.owner_of(i)])
    return ModelSpec(width=d, vocab_size=cfg.vocab, token_table="embed",
                     position=PartSpec("learned_absolute", "", {"width": d, "n_positions": cfg.max_positions, "table": "pos"}),
                     layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"), head="head",
                     embedding_scale=cfg.embedding_scale, scale_positions=False, logit_scale=cfg.logit_scale)


register_architecture(SosutarConfig.architecture, SosutarConfig, build_spec)
