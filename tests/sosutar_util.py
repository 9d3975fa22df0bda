"""Small Sosutar configurations and helpers shared by the CPU and GPU tests.

The configurations differ from one another in every size and option: an mLSTM with values wider than keys
and one with keys wider than values, with and without a feed-forward behind it; attention with grouped heads
and values wider than keys / plain heads with equal sizes; a window shorter than a page / longer than a page;
a query temperature that steps every few positions / once in the test's lengths; layers that run with the
tensors of an earlier or of a later layer; a third model whose sizes are no multiples of 8 anywhere, with one
head, a factor of one on the embedding and on the logits, and a soft cap so wide that it hardly bends the gates.
"""
import copy
import json
import os

import numpy as np


def _mlstm(heads, dim, vdim, cap, mlp=None, **more):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp, **more}


def _parallel(left, right_width, mlp, **more):
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": right_width}}, "mlp": mlp, **more}


LEFT_A = {"dim": 16, "vdim": 32, "heads": 4, "kv_heads": 2, "scale": 0.31, "mask": {"size": 20}, "q_temp": {"coef": 0.4, "every": 8}}
LEFT_B = {"dim": 32, "vdim": 32, "heads": 3, "kv_heads": 3, "scale": 0.15, "mask": {"size": 70}, "q_temp": {"coef": 1.5, "every": 64}}
LEFT_C = {"dim": 12, "vdim": 10, "heads": 3, "kv_heads": 1, "scale": 0.25, "mask": {"size": 9}, "q_temp": {"coef": 0.0, "every": 1}}
DENSE = lambda ff: {"kind": "dense", "ff": ff}  # noqa: E731

CONFIGS = {
    "sos_a": {"architecture": "Sosutar", "vocab": 300, "width": 64, "max_positions": 700, "norm": {"eps": 1e-5},
              "embedding": {"scale": 4.0}, "logit_scale": 0.25, "layers": [
                  _mlstm(2, 16, 24, 6.0),
                  _parallel(LEFT_A, 40, DENSE(104)),
                  _mlstm(2, 16, 24, 6.0, weights_of=0),
                  _parallel(LEFT_A, 40, None),
                  _parallel(LEFT_A, 40, DENSE(104), weights_of=1)]},
    "sos_b": {"architecture": "Sosutar", "vocab": 200, "width": 96, "max_positions": 512, "norm": {"eps": 1e-6},
              "embedding": {"scale": 0.5}, "logit_scale": 2.0, "layers": [
                  _parallel(LEFT_B, 136, DENSE(160), weights_of=2),
                  _mlstm(3, 32, 16, 3.0, DENSE(48)),
                  _parallel(LEFT_B, 136, DENSE(160))]},
    "sos_c": {"architecture": "Sosutar", "vocab": 101, "width": 60, "max_positions": 300, "norm": {"eps": 1e-5},
              "embedding": {"scale": 1.0}, "logit_scale": 1.0, "layers": [
                  _parallel(LEFT_C, 50, DENSE(50)),
                  _mlstm(1, 12, 10, 30.0)]},
}
SEEDS = {"sos_a": 3, "sos_b": 4, "sos_c": 5}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def write_model(folder: str, cfg: dict, seed: int, scale_up: float = 6.0) -> str:
    """A model folder with random weights through the library's own random-weights mode, the matrices
    scaled up so that attention and the recurrences matter in the logits."""
    import torch

    import ember_cpp_b200 as E
    from ember_cpp_b200.weights import read_folder, write_file
    E.write_random_model(folder, E.config.config_from_dict(cfg), seed)
    tensors = {name: t.clone() for name, t in read_folder(folder).items()}     # (the file is mapped: copies, then rewrite)
    for name, t in tensors.items():
        if t.dtype.is_floating_point and t.dim() == 2:
            tensors[name] = (t.float() * (2.0 if name in ("embed", "head", "pos") else scale_up)).to(torch.bfloat16)
    write_file(os.path.join(folder, "model.safetensors"), tensors, {"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return folder


def ids(seed: int, vocab: int, n: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def steady_tokens(m) -> list:
    """Tokens that a test sequence may begin with.  At a sequence's first position the matrix memory holds one term, so
    a head's read-out is its value times the sign of k . q (the head's norm takes the size away); for a token whose
    k . q happens to lie near zero in some head of some layer, a rounding of q or k in bfloat16 decides that sign, and no
    tolerance on the logits is meaningful.  These are the tokens whose |k . q| / (|k| |q|) is above 0.1 in every
    head of every such layer, by the plain model `m`."""
    import plain_sosutar as P
    cfg, eps = m.cfg, m.cfg["norm"]["eps"]
    steady = []
    for tok in range(cfg["vocab"]):
        x = m.w["embed"][[tok]] * cfg["embedding"]["scale"] + m.w["pos"][:1]
        worst = 1.0
        for i, layer in enumerate(cfg["layers"]):
            if layer["type"] == "mlstm":
                p, c = f"l{layer.get('weights_of', i)}.mix.", layer["mixer"]
                h = P.rms_norm(x, m.w[p[:-4] + "norm1"], eps)
                q, k = ((h @ m.w[p + n].T).reshape(c["heads"], c["dim"]) for n in ("q", "k"))
                worst = min(worst, (np.abs((q * k).sum(-1)) / (np.linalg.norm(q, axis=1) * np.linalg.norm(k, axis=1))).min())
            x = P.layer(m, i, x)
        if worst > 0.1:
            steady.append(tok)
    return steady


def sequences(m, seed: int, lengths) -> list:
    """Random sequences of the given lengths for the plain model `m`, each beginning with a steady token."""
    steady = steady_tokens(m) if not hasattr(m, "_steady") else m._steady
    m._steady = steady
    out = []
    for i, n in enumerate(lengths):
        seq = ids(seed + i, m.cfg["vocab"], n)
        seq[0] = steady[(seed + i) % len(steady)]
        out.append(seq)
    return out


def row_error(got, ref) -> float:
    """Worst row of rms(delta - mean(delta)) / rms(ref - mean(ref))."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if ref.ndim == 1:
        got, ref = got[None], ref[None]
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1))).max())


# of a row's spread (see row_error).  bfloat16: these models' weights are scaled up so that every mechanism shows in
# the logits, which also lets the roundings of activations through: the engine is within this of the exact rows
TOL = {"float32": 3e-5, "bfloat16": 8e-2}
