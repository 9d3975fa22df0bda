"""Vipolix, slowly: numpy in float64, one function per mechanism, whole sequences, no cache.

It shares no code with the library: it reads config.json as a plain dict and model.safetensors with
a reader of its own, and walks every recurrence token by token.  The tests compare the library's
kernels, its step function and its generation loop with these functions.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ------------------------------------------------------------------------------------------ files
def read_safetensors(path):
    """name -> float64 array (integer tables as int64)."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, shape = data[lo:hi], tuple(info["shape"])
        kind = info["dtype"]
        if kind == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif kind == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif kind == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: element type {kind}")
        out[name] = a.reshape(shape)
    return out


def load_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ------------------------------------------------------------------------------------------ small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """Rows divided by their root mean square, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_around_zero(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


def token_shift(h, mu, before=None):
    """h[t] + (h[t-1] - h[t]) * mu, the row before the first being `before` (zeros at a sequence's start)."""
    prev = np.zeros_like(h)
    prev[1:] = h[:-1]
    if before is not None:
        prev[0] = before
    return h + (prev - h) * mu


def short_conv(u, w):
    """Causal convolution over time, a filter a channel: y[t] = sum_j w[:, j] u[t - taps + 1 + j]; u [T, C], w [C, taps]."""
    T, taps = u.shape[0], w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u])
    y = np.zeros_like(u)
    for j in range(taps):
        y += padded[j:j + T] * w[:, j]
    return y


def rotate_pairs(x, positions, dims, base):
    """x [T, heads, dim]: the first `dims` of every head rotated, neighbours (2i, 2i+1) as a pair."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = positions[:, None].astype(np.float64) * base ** (-2.0 * i / dims)        # [T, dims/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ------------------------------------------------------------------------------------------ mixers
def gla_recurrence(q, k, v, alpha, S=None):
    """q, k, alpha [T, H, D]; v [T, H, V].  S <- diag(alpha) S + k v^T; o = S^T q.  Returns o [T, H, V] and the last S."""
    T, H, D = q.shape
    V = v.shape[2]
    S = np.zeros((H, D, V)) if S is None else S.copy()
    o = np.zeros((T, H, V))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    return o, S


def gla_mixer(h, W, p, m, eps):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, V)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = sigmoid(z).reshape(T, H, D) ** (1.0 / m["tau"])
    o, _ = gla_recurrence(q, k, v, alpha)
    o = norm_plain(o, W[p + "norm"], eps).reshape(T, H * V)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def chunked_sink_attention(q, k, v, positions, scale, temps, size):
    """q [T, H, D]; k [T, G, D]; v [T, G, V]; keys are the sequence's own rows.  A query at position i sees the keys
    j <= i of its own chunk of `size` positions; the softmax's denominator holds one more 1."""
    T, H, D = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * scale * temps[hh]
        pi, pj = positions[:, None], positions[None, :]
        seen = (pj <= pi) & (pi // size == pj // size)
        s = np.where(seen, s, -np.inf)
        top = np.maximum(s.max(axis=1, keepdims=True), 0.0)
        e = np.exp(s - top)
        out[:, hh] = (e @ v[:, g]) / (np.exp(-top) + e.sum(axis=1, keepdims=True))
    return out


def left_mixer(h, W, p, m, positions):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    rows = {}
    for n in ("q", "k", "v"):
        rows[n] = short_conv(h @ W[p + n].T + W[p + n + ".b"], W[p + n + ".conv"])
    q = rotate_pairs(rows["q"].reshape(T, H, D), positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_pairs(rows["k"].reshape(T, G, D), positions, m["rot"]["dims"], m["rot"]["base"])
    v = rows["v"].reshape(T, G, V)
    o = chunked_sink_attention(q, k, v, positions, m["scale"], W[p + "temp"], m["mask"]["size"])
    return o.reshape(T, H * V) @ W[p + "o"].T


def delta_recurrence(r, k, v, w, a, S=None):
    """All [T, H, D].  With u = k / sqrt(sum k^2 + 1e-6):  S <- diag(w) S - (a u)(u^T S) + k v^T, both of the first
    two terms reading the state of the token before; o = S^T r."""
    T, H, D = r.shape
    S = np.zeros((H, D, D)) if S is None else S.copy()
    o = np.zeros((T, H, D))
    for t in range(T):
        u = k[t] / np.sqrt(np.sum(k[t] ** 2, axis=-1, keepdims=True) + 1e-6)
        uS = np.einsum("hd,hdv->hv", u, S)
        S = w[t][:, :, None] * S - (a[t] * u)[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, r[t])
    return o, S


def right_mixer(h, W, p, m, eps):
    H, D = m["heads"], m["dim"]
    T = h.shape[0]
    r, k, v = ((h @ W[p + n].T).reshape(T, H, D) for n in ("r", "k", "v"))
    w = np.exp(-math.exp(-0.5) * sigmoid(np.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, H, D)
    a = sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).reshape(T, H, D)
    o, _ = delta_recurrence(r, k, v, w, a)
    o = unit_rms(o, eps).reshape(T, H * D) * W[p + "norm"]
    return (o * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ feed-forward
def clamped_expert(h, gate, up, down, limit):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, W, p, r):
    """Chosen experts [T, top] and their weights [T, top]."""
    E, top = r["experts"], r["top"]
    s = sigmoid(h @ W[p + "router"].T)
    choice = s + W[p + "correction"]
    groups = r.get("groups")
    if groups:
        per = E // groups["count"]
        grouped = choice.reshape(-1, groups["count"], per)
        best2 = np.sort(grouped, axis=-1)[..., -2:].sum(axis=-1) if per >= 2 else grouped.sum(axis=-1)
        order = np.argsort(-best2, axis=-1, kind="stable")[:, :groups["keep"]]
        allowed = np.zeros((h.shape[0], groups["count"]), dtype=bool)
        np.put_along_axis(allowed, order, True, axis=1)
        choice = np.where(np.repeat(allowed, per, axis=1), choice, -np.inf)
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    weights = np.take_along_axis(s, chosen, axis=1)
    weights = weights / (weights.sum(axis=1, keepdims=True) + 1e-20) * r["scale"]
    return chosen, weights


def experts_ff(h, W, p, mlp):
    chosen, weights = route(h, W, p, mlp["router"])
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            q = f"{p}e{e}."
            out[t] += wt * clamped_expert(h[t:t + 1], W[q + "gate"], W[q + "up"], W[q + "down"], mlp["expert"]["limit"])[0]
    shared = mlp.get("shared")
    if shared:
        q = p + "shared."
        out += sigmoid(h @ W[q + "sg"].T) * clamped_expert(h, W[q + "gate"], W[q + "up"], W[q + "down"], shared["limit"])
    return out


def side_input(x, tokens, W, p, layer, dim, eps):
    e = W["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ W[p + "side.gate"].T) * e) @ W[p + "side.proj"].T
    return norm_plain(y, W[p + "side.norm"], eps)


# ------------------------------------------------------------------------------------------ the model
def forward(cfg, W, tokens, per_layer=False):
    """Logits [T, vocab] of one sequence from its first token; with `per_layer` also the stream after every layer."""
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = np.arange(len(tokens))
    eps = cfg["norm"]["eps"]
    x = W["embed"][tokens]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = token_shift(norm_around_zero(x, W[p + "norm1"], eps), W[p + "shift"])
        m = layer["mixer"]
        if layer["type"] == "gla":
            x = x + gla_mixer(h, W, p + "mix.", m, eps)
        else:
            x = x + m["left_scale"] * left_mixer(h, W, p + "mix.left.", m["left"], positions) \
                + m["right_scale"] * right_mixer(h, W, p + "mix.right.", m["right"], eps)
        if layer.get("mlp") is not None:
            x = x + experts_ff(norm_around_zero(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
        if cfg.get("token_side"):
            x = x + side_input(x, tokens, W, p, i, cfg["token_side"]["dim"], eps)
        streams.append(x.copy())
    logits = norm_around_zero(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.stack(streams)) if per_layer else logits


def generate(cfg, W, prompt, steps):
    """Greedy continuation: the first of the largest logits, `steps` times."""
    ids = list(prompt)
    for _ in range(steps):
        ids.append(int(np.argmax(forward(cfg, W, ids)[-1])))
    return ids[len(prompt):]
