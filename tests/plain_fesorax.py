"""A plain, slow statement of the Fesorax decoder: one function per mechanism, NumPy float64,
whole sequences, no cache, no batching.  It shares no code with the library under test.

The design: a post-norm residual stream (x <- norm(alpha x + sublayer(x))), mixers that are
either gated softmax attention with unit-norm queries and keys, a learned bias by log-bucketed
distance and a sliding window that keeps the first tokens (optionally on another layer's keys
and values), or an mLSTM matrix memory with a stabilised exponential gate; and feed-forwards
that are mixtures of clamped gated experts whose router weight scales the expert's input, plus
a shared expert.

``round_fn`` rounds what a bfloat16 engine stores in bfloat16 (projections, activations, cached
keys and values); the residual, scores, softmax weights, gates, norms, routers and recurrent
state stay unrounded, as they do there.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np


def _id(a):
    return a


# ---- small pieces ------------------------------------------------------------------------------
def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return unit_rms(x, eps) * w


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z: np.ndarray) -> np.ndarray:
    return -np.logaddexp(0.0, -z)


def softmax_rows(s: np.ndarray) -> np.ndarray:
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


# ---- attention mixer ---------------------------------------------------------------------------
def distance_bucket(n: int, n_buckets: int, max_distance: int) -> int:
    """Distances below half the table are their own bucket; beyond, buckets grow logarithmically up
    to ``max_distance`` and the last bucket takes the rest.  The logarithms are single precision."""
    half = n_buckets // 2
    if n < half:
        return n
    t = np.float32(np.log(np.float32(n) / np.float32(half))) / np.float32(math.log(max_distance / half))
    return min(n_buckets - 1, half + int(np.floor(np.float32(t) * np.float32(n_buckets - half))))


def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j (window 0: every earlier key)."""
    return j <= i and (window <= 0 or i - j < window or j < keep_first)


def attention_keys_values(h, w, p, m, eps, r=_id):
    """Keys after their unit norm, and values, as the layer's cache would hold them."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = r(h @ w[p + "k"].T).reshape(T, G, d)
    v = r(h @ w[p + "v"].T).reshape(T, G, dv)
    return r(unit_rms(k, eps)), v


def attention_mixer(h, w, p, m, eps, k, v, r=_id):
    """h [T, width] -> [T, width].  ``k``/``v`` are this layer's own or another layer's."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mask = m.get("mask") or {}
    window, keep = int(mask.get("size", 0)), int(mask.get("keep_first", 0))
    q = unit_rms(r(h @ w[p + "q"].T).reshape(T, H, d), eps)
    q = r(q)
    rel = w[p + "rel"]
    B = rel.shape[0]
    gate = sigmoid(h @ w[p + "g"].T)  # [T, H]
    out = np.zeros((T, H, dv))
    bucket_of = np.array([distance_bucket(n, B, m["bias_max"]) for n in range(T)])
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = np.array([[visible(a, b, window, keep) for b in range(T)] for a in range(T)]) if T <= 64 else \
        (j <= i) & ((window <= 0) | (i - j < window) | (j < keep))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] + rel[bucket_of[np.maximum(i - j, 0)], hd]
        out[:, hd] = softmax_rows(np.where(seen, s, -np.inf)) @ v[:, g]
    out = r(out * gate[:, :, None])
    return r(out.reshape(T, H * dv) @ w[p + "o"].T)


# ---- mLSTM mixer -------------------------------------------------------------------------------
def mlstm_gates(h, w, p, m):
    """Log input gate and log forget gate per token and head, both soft-capped."""
    cap = m["gate_cap"]
    i = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    f = log_sigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    return i, f


def mlstm_recurrence(q, k, v, i, f):
    """q, k [T, H, d], v [T, H, dv], gates [T, H] -> [T, H, dv], token by token."""
    T, H, d = q.shape
    dv = v.shape[2]
    out = np.zeros((T, H, dv))
    for hd in range(H):
        S, n, mx = np.zeros((d, dv)), np.zeros(d), 0.0
        for t in range(T):
            m_new = max(f[t, hd] + mx, i[t, hd])
            a, b = math.exp(f[t, hd] + mx - m_new), math.exp(i[t, hd] - m_new)
            S = a * S + b * np.outer(k[t, hd], v[t, hd])
            n = a * n + b * k[t, hd]
            mx = m_new
            out[t, hd] = (S.T @ q[t, hd]) / (max(abs(float(n @ q[t, hd])), math.exp(-mx)) + 1e-6)
    return out


def mlstm_mixer(h, w, p, m, eps, r=_id):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = r(h @ w[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = r(h @ w[p + "k"].T).reshape(T, H, d)
    v = r(h @ w[p + "v"].T).reshape(T, H, dv)
    i, f = mlstm_gates(h, w, p, m)
    o = unit_rms(mlstm_recurrence(q, k, v, i, f), eps).reshape(T, H * dv)
    o = r(o * w[p + "norm"] * sigmoid(r(h @ w[p + "g"].T)))
    return r(o @ w[p + "o"].T)


# ---- feed-forward ------------------------------------------------------------------------------
def expert(h, w, p, limit, r=_id):
    """down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate h, limit), u = clamp(up h, +-limit)."""
    g = np.minimum(r(h @ w[p + "gate"].T), limit)
    u = np.clip(r(h @ w[p + "up"].T), -limit, limit)
    return r(r(g * sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T)


def route(h, w_router, top):
    """Per token the ``top`` experts with the largest sigmoid scores, and those scores."""
    s = sigmoid(h @ w_router.T)
    idx = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1)


def moe(h, w, p, mlp, r=_id):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, score = route(h, w[p + "router"], top)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, s in zip(idx[t], score[t]):
            out[t] += expert(r(s * h[t:t + 1]), w, f"{p}e{e}.", mlp["expert"]["limit"], r)[0]
    if mlp.get("shared"):
        out += expert(h, w, p + "shared.", mlp["shared"]["limit"], r)
    return out


# ---- the model ---------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], round_fn=None,
            residuals: Optional[List[np.ndarray]] = None) -> np.ndarray:
    """Logits [T, vocab]; with ``residuals`` the stream after every layer is appended to it."""
    r = round_fn or _id
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    kept = {}
    for li, layer in enumerate(cfg["layers"]):
        p, m = f"l{li}.mix.", layer["mixer"]
        h = r(x)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[li] = attention_keys_values(h, w, p, m, eps, r)
                src = li
            y = attention_mixer(h, w, p, m, eps, *kept[src], r)
        elif layer["type"] == "mlstm":
            y = mlstm_mixer(h, w, p, m, eps, r)
        else:
            raise ValueError(layer["type"])
        x = rms_norm(alpha * x + y, w[f"l{li}.norm1"], eps)
        if layer.get("mlp"):
            x = rms_norm(alpha * x + moe(r(x), w, f"l{li}.mlp.", layer["mlp"], r), w[f"l{li}.norm2"], eps)
        elif f"l{li}.norm2" in w:
            x = rms_norm(alpha * x, w[f"l{li}.norm2"], eps)
        if residuals is not None:
            residuals.append(x.copy())
    return r(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
