"""Plain Sosutar: whole sequences, no cache, no state carried between calls, one function for
each mechanism.

Sosutar is a pre-norm decoder with a learned position table and a per-channel gain on every
sublayer's output.  Its layers are of two kinds: a matrix-memory recurrence (mLSTM) without a
feed-forward, and two mixers side by side on the same input, a sliding-window attention (norms on
q, k and v, a query temperature that grows with the position, a linear distance penalty, a sink in
the softmax's denominator, an output gate) and a minGRU recurrence, each output normed before
their mean is taken.  A layer may run with another layer's tensors.  Feed-forwards are dense with
a squared relu.

Nothing here is shared with the engine: own safetensors reader, own arithmetic (numpy, float64),
loops over tokens where the definition is a recurrence.  It is the exact value that the engine's
float32 and bfloat16 paths approximate.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

DENOMINATOR_FLOOR = 1e-6     # added to the mLSTM read-out's denominator
SLOPE_BASE = 8.0             # distance slopes are 2^(-SLOPE_BASE (h + 1) / heads)


# --------------------------------------------------------------------------- model folder
def read_safetensors(path: str) -> dict[str, np.ndarray]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        kind = meta["dtype"].upper()
        if kind == "BF16":
            a = (np.frombuffer(data[b:e], dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif kind == "F32":
            a = np.frombuffer(data[b:e], dtype="<f4").astype(np.float64)
        elif kind == "I32":
            a = np.frombuffer(data[b:e], dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"plain reader: dtype {kind} of {name}")
        out[name] = a.reshape(meta["shape"])
    return out


class PlainSosutar:
    def __init__(self, folder: str | None = None, cfg: dict | None = None, weights: dict | None = None):
        if folder is not None:
            with open(os.path.join(folder, "config.json")) as f:
                cfg = json.load(f)
            weights = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.cfg, self.w = cfg, weights


# --------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    """Rows divided by sqrt(mean of squares + eps)."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return rms_unit(x, eps) * w


def soft_cap(z, cap: float):
    return cap * np.tanh(z / cap)


# --------------------------------------------------------------------------- the matrix memory
def mlstm_recurrence(q, k, v, log_i, log_f):
    """One head.  q, k [T, dim] (q already scaled), v [T, vdim], log_i and log_f [T].  The memory S, its
    normaliser n and the running maximum m all start at zero."""
    T, dim = q.shape
    S = np.zeros((dim, v.shape[1]))
    n = np.zeros(dim)
    m = 0.0
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        m_new = max(log_f[t] + m, log_i[t])
        keep, take = math.exp(log_f[t] + m - m_new), math.exp(log_i[t] - m_new)
        S = keep * S + take * np.outer(k[t], v[t])
        n = keep * n + take * k[t]
        m = m_new
        out[t] = (S.T @ q[t]) / (max(abs(n @ q[t]), math.exp(-m)) + DENOMINATOR_FLOOR)
    return out


def mlstm(h, w, heads, dim, vdim, cap, eps):
    """w: the mixer's tensors by their short names (q, k, v, g, o, norm, i, i.b, f, f.b)."""
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, heads, dim) * dim ** -0.5
    k = (h @ w["k"].T).reshape(T, heads, dim)
    v = (h @ w["v"].T).reshape(T, heads, vdim)
    log_i = soft_cap(h @ w["i"].T + w["i.b"], cap)
    log_f = log_sigmoid(soft_cap(h @ w["f"].T + w["f.b"], cap))
    o = np.stack([rms_unit(mlstm_recurrence(q[:, a], k[:, a], v[:, a], log_i[:, a], log_f[:, a]), eps)
                  for a in range(heads)], axis=1).reshape(T, heads * vdim)
    return (o * w["norm"] * sigmoid(h @ w["g"].T)) @ w["o"].T


# --------------------------------------------------------------------------- the attention
def temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def slope(head: int, heads: int) -> float:
    return 2.0 ** (-SLOPE_BASE * (head + 1) / heads)


def sink_attention(h, w, heads, kv_heads, dim, vdim, scale, window, coef, every, eps):
    """w: q, k, v, q.norm, k.norm, sink, g, o."""
    T = h.shape[0]
    q = rms_norm(h @ w["q"].T, w["q.norm"], eps)             # over the whole projection, before the heads are cut
    k = rms_norm(h @ w["k"].T, w["k.norm"], eps)
    q = q * np.array([temperature(p, coef, every) for p in range(T)])[:, None]
    q = q.reshape(T, heads, dim)
    k = k.reshape(T, kv_heads, dim)
    v = rms_unit((h @ w["v"].T).reshape(T, kv_heads, vdim), eps)
    out = np.zeros((T, heads, vdim))
    per = heads // kv_heads
    for a in range(heads):
        g = a // per
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, a]) * scale - slope(a, heads) * (i - np.arange(lo, i + 1))
            top = max(s.max(), w["sink"][a])
            e = np.exp(s - top)
            out[i, a] = (e @ v[lo:i + 1, g]) / (e.sum() + math.exp(w["sink"][a] - top))
    return (out.reshape(T, heads * vdim) * sigmoid(h @ w["g"].T)) @ w["o"].T


# --------------------------------------------------------------------------- the small recurrence
def mingru_candidate(u):
    return np.where(u >= 0, u + 0.5, sigmoid(u))


def mingru(h, w):
    """w: z, z.b, x, x.b, g, o."""
    z = sigmoid(h @ w["z"].T + w["z.b"])
    c = mingru_candidate(h @ w["x"].T + w["x.b"])
    S = np.zeros(z.shape[1])
    states = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        states[t] = S
    return (states * silu(h @ w["g"].T)) @ w["o"].T


# --------------------------------------------------------------------------- feed-forward
def relu2_dense(h, w_up, w_down):
    return np.square(np.maximum(h @ w_up.T, 0.0)) @ w_down.T


# --------------------------------------------------------------------------- the model
def _sub(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in weights.items() if name.startswith(prefix)}


def mixer(m: PlainSosutar, entry: dict, prefix: str, h):
    eps = m.cfg["norm"]["eps"]
    c = entry["mixer"]
    if entry["type"] == "mlstm":
        return mlstm(h, _sub(m.w, prefix + "mix."), c["heads"], c["dim"], c["vdim"], c["gate_cap"], eps)
    if entry["type"] == "parallel":
        a = c["left"]
        left = sink_attention(h, _sub(m.w, prefix + "mix.left."), a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["scale"],
                              a["mask"]["size"], a["q_temp"]["coef"], a["q_temp"]["every"], eps)
        right = mingru(h, _sub(m.w, prefix + "mix.right."))
        return 0.5 * (rms_norm(left, m.w[prefix + "mix.left.out"], eps) + rms_norm(right, m.w[prefix + "mix.right.out"], eps))
    raise ValueError(f"plain model: layer type {entry['type']!r}")


def layer(m: PlainSosutar, i: int, x):
    entry, owner = m.cfg["layers"][i], i
    while m.cfg["layers"][owner].get("weights_of") is not None:       # (a layer named there may name another in turn)
        owner = m.cfg["layers"][owner]["weights_of"]
    p = f"l{owner}."
    eps = m.cfg["norm"]["eps"]
    x = x + m.w[p + "ls1"] * mixer(m, entry, p, rms_norm(x, m.w[p + "norm1"], eps))
    if entry.get("mlp") is not None:
        h = rms_norm(x, m.w[p + "norm2"], eps)
        x = x + m.w[p + "ls2"] * relu2_dense(h, m.w[p + "mlp.up"], m.w[p + "mlp.down"])
    return x


def forward(m: PlainSosutar, ids, streams: list | None = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence from its first token; `streams` collects the residual stream after every layer."""
    ids = np.asarray(ids)
    x = m.w["embed"][ids] * m.cfg["embedding"]["scale"] + m.w["pos"][:len(ids)]
    for i in range(len(m.cfg["layers"])):
        x = layer(m, i, x)
        if streams is not None:
            streams.append(x.copy())
    return rms_norm(x, m.w["final.norm"], m.cfg["norm"]["eps"]) @ m.w["head"].T * m.cfg["logit_scale"]


def generate(m: PlainSosutar, prompt, n_new: int) -> list[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(np.argmax(forward(m, ids)[-1])))
    return ids[len(prompt):]
