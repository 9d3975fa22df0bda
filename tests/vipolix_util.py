"""Small Vipolix configurations and helpers shared by the CPU and GPU tests.

The configurations differ from one another in every size and option: gated linear attention with values wider
and narrower than keys, one head and several, a tau of 1 and larger ones; the attention beside the delta rule
with grouped and plain heads, values of the keys' size and of another, convolutions of 4, 2 and 1 taps (the last
carries no state), a chunk shorter than a page, longer than a page (and no multiple of it) and very short, a part of
every head rotated or all of it; experts with and without groups, with and without a shared expert, all experts
chosen or one; layers without a feed-forward; with and without the per-layer input from the token ids; a third
model whose sizes are no multiples of 8 anywhere, with a factor below zero on one attention head's scores.
"""
import copy
import json
import os

import numpy as np


def _left(dim, vdim, heads, kv, conv, chunk, rot_dims, base, scale):
    return {"dim": dim, "vdim": vdim, "heads": heads, "kv_heads": kv, "conv": conv, "mask": {"size": chunk},
            "rot": {"dims": rot_dims, "base": base}, "scale": scale}


def _moe(experts, top, ff, limit, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


def _gla(heads, dim, vdim, tau, mlp, rank=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    if rank:
        m["decay_rank"] = rank
    return {"type": "gla", "mixer": m, "mlp": mlp}


def _parallel(left, right_dim, right_heads, scales, mlp, rank=None):
    right = {"dim": right_dim, "heads": right_heads}
    if rank:
        right["decay_rank"] = rank
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": scales[0], "right_scale": scales[1]}, "mlp": mlp}


LEFT_A = _left(32, 32, 4, 2, 4, 20, 16, 10000.0, 0.2)
LEFT_B = _left(16, 48, 3, 3, 1, 70, 16, 100.0, 0.3)
LEFT_C = _left(12, 10, 3, 1, 2, 9, 4, 50.0, 0.35)

CONFIGS = {
    "vip_a": {"architecture": "Vipolix", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8}, "layers": [
        _parallel(LEFT_A, 16, 2, (0.7, 1.3), _moe(8, 2, 24, 1.5, 1.5, groups=(4, 2), shared=(40, 3.0))),
        _gla(2, 16, 24, 4.0, None),
        _parallel(LEFT_A, 16, 2, (0.7, 1.3), _moe(8, 3, 24, 1.5, 1.0)),
        _gla(2, 16, 24, 4.0, _moe(4, 1, 16, 2.5, 2.0, groups=(2, 1)), rank=5)]},
    "vip_b": {"architecture": "Vipolix", "vocab": 200, "width": 96, "norm": {"eps": 1e-6}, "layers": [
        _gla(3, 32, 16, 1.0, _moe(6, 6, 32, 1.0, 1.0)),
        _parallel(LEFT_B, 48, 1, (1.0, 0.5), _moe(6, 2, 32, 4.0, 2.5, groups=(3, 3), shared=(16, 0.5)), rank=24),
        _parallel(LEFT_B, 48, 1, (1.0, 0.5), None)]},
    "vip_c": {"architecture": "Vipolix", "vocab": 101, "width": 60, "norm": {"eps": 1e-5}, "token_side": {"dim": 5}, "layers": [
        _gla(1, 12, 10, 2.5, _moe(5, 1, 14, 2.0, 1.0, shared=(6, 2.0)), rank=3),
        _parallel(LEFT_C, 12, 2, (1.5, 1.0), _moe(5, 2, 14, 2.0, 3.0))]},
}
SEEDS = {"vip_a": 3, "vip_b": 4, "vip_c": 5}
TOL = {"float32": 1e-4, "bfloat16": 8e-2}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def write_model(folder: str, cfg: dict, seed: int, scale_up: float = 6.0) -> str:
    """A model folder with random weights through the library's own random-weights mode, the matrices
    scaled up so that the mixers and the experts matter in the logits; in `vip_c` one head's factor on its
    scores is made negative."""
    import torch

    import ember_cpp_b200 as E
    from ember_cpp_b200.weights import read_folder, write_file
    E.write_random_model(folder, E.config.config_from_dict(cfg), seed)
    tensors = {name: t.clone() for name, t in read_folder(folder).items()}     # (the file is mapped: copies, then rewrite)
    for name, t in tensors.items():
        if not t.dtype.is_floating_point or t.dim() != 2:
            continue
        if name in ("embed", "head"):
            tensors[name] = (t.float() * 2.0).to(torch.bfloat16)
        elif not name.endswith((".conv", ".a2", ".w2", ".router", "side.embed")):
            tensors[name] = (t.float() * scale_up).to(torch.bfloat16)
    if cfg["width"] == 60:
        tensors["l1.mix.left.temp"][1] = -0.75
    if cfg["width"] == 64:      # routers whose scores lie close together: the stored corrections decide most choices, so
        for name in tensors:    # that few choices are near ties that a rounding in bfloat16 turns the other way
            if name.endswith(".router"):
                tensors[name] = (tensors[name].float() * 0.1).to(torch.bfloat16)
    write_file(os.path.join(folder, "model.safetensors"), tensors, {"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return folder


def ids(seed: int, vocab: int, n: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def rows_agree(got, ref, dtype: str) -> bool:
    """`got` against the plain model's `ref` (lists of [rows, vocab] arrays).  In 32-bit every row is within TOL.  In
    bfloat16 a rounding can turn a near tie of the router's choice the other way, and the token then runs another expert
    than the plain model's: some rows may differ by more (at most one in five; measured: one in eight with eight experts in
    three layers, none with five experts in one), the typical row must not."""
    errors = np.array([row_error(g[i], r[i]) for g, r in zip(got, ref) for i in range(len(r))])
    if dtype == "float32":
        return bool(errors.max() < TOL[dtype])
    return bool((errors >= TOL[dtype]).mean() <= 0.2 and np.median(errors) < TOL[dtype] / 2)


def row_error(got, ref) -> float:
    """Worst row of rms(delta - mean(delta)) / rms(ref - mean(ref))."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if ref.ndim == 1:
        got, ref = got[None], ref[None]
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    return float((np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1))).max())
