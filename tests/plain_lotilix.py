"""A plain, slow statement of the Lotilix decoder: one function per mechanism, NumPy float64,
whole sequences, no cache, no batching.  It shares no code with the library under test.

The design: parallel blocks (one norm whose output both the mixer and the feed-forward read, their
sum added to the stream), followed in every layer by a small gated input looked up by token id;
mixers that are softmax attention through low-rank latents with a shared rotated key part, a
sliding window and a gate per head, or grouped-query attention whose values are its unrotated keys
and whose mask is cut into chunks, or a gated delta rule with one decay per key channel; and a
dense feed-forward with the tanh form of GELU.

``round_fn`` rounds what a bfloat16 engine stores in bfloat16 (projections, activations, cached
rows); the residual, scores, softmax weights, gates, decays, norms and recurrent state stay
unrounded, as they do there.
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import numpy as np


def _id(a):
    return a


def to_bf16(a):
    """Round to the nearest bfloat16 (ties to even), returned as float64."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


# ---- small pieces ------------------------------------------------------------------------------
def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softmax_masked(s, seen):
    s = np.where(seen, s, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


# ---- positions ---------------------------------------------------------------------------------
def rotary_frequencies(rot: dict) -> np.ndarray:
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` long wavelengths are slowed: beyond
    original/low by ``factor``, between original/high and original/low by a blend."""
    dims = int(rot["dims"])
    f = float(rot["base"]) ** (-2.0 * np.arange(dims // 2) / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wl = 2.0 * math.pi / fi
            if wl < orig / high:
                out.append(fi)
            elif wl > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wl - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = np.array(out)
    return f


def rotate_pairs(x, positions, freqs):
    """x [T, heads, d]: the pairs (2i, 2i+1), i < len(freqs), are turned by positions * freqs[i]."""
    out = x.copy()
    n = len(freqs)
    a = np.asarray(positions, dtype=np.float64)[:, None, None] * freqs[None, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * np.cos(a) - v * np.sin(a)
    out[..., 1:2 * n:2] = v * np.cos(a) + u * np.sin(a)
    return out


# ---- masks -------------------------------------------------------------------------------------
def sees_window(i: int, j: int, size: int) -> bool:
    return 0 <= i - j and (size <= 0 or i - j < size)


def sees_chunk(i: int, j: int, size: int) -> bool:
    return j <= i and (size <= 0 or i // size == j // size)


def mask_matrix(T: int, size: int, rule) -> np.ndarray:
    return np.array([[rule(i, j, size) for j in range(T)] for i in range(T)], dtype=bool)


# ---- mixers ------------------------------------------------------------------------------------
def latent_attention(h, w, p, m, eps, r=_id):
    """Queries through a normed latent; keys and values from one normed latent per token plus one
    rotated key part shared by all heads; sliding window; a logistic gate per head."""
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    freqs = rotary_frequencies(m["rot"])
    cq = r(rms_norm(r(h @ w[p + "dq"].T), w[p + "dq.norm"], eps))
    q = r(cq @ w[p + "uq"].T).reshape(T, H, d + dr)
    q_plain, q_rot = q[..., :d], r(rotate_pairs(q[..., d:], pos, freqs))
    dkv = r(h @ w[p + "dkv"].T)
    c = r(rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps))
    k_rot = r(rotate_pairs(dkv[:, None, rank:], pos, freqs))[:, 0]
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    seen = mask_matrix(T, int((m.get("mask") or {}).get("size", 0)), sees_window)
    gate = sigmoid(r(h @ w[p + "g"].T))
    out = np.zeros((T, H, dv))
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        out[:, a] = (softmax_masked(s, seen) @ v[:, a]) * gate[:, a:a + 1]
    return r(out.reshape(T, H * dv)) @ w[p + "o"].T


def chunked_attention(h, w, p, m, eps, r=_id):
    """Grouped-query attention whose values are the keys before rotation; a query sees the earlier
    keys of its own chunk of ``mask.size`` positions."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = np.arange(T)
    freqs = rotary_frequencies(m["rot"])
    q = r(rotate_pairs(r(h @ w[p + "q"].T).reshape(T, H, d), pos, freqs))
    v = r(h @ w[p + "k"].T).reshape(T, G, d)
    k = r(rotate_pairs(v, pos, freqs))
    seen = mask_matrix(T, int((m.get("mask") or {}).get("size", 0)), sees_chunk)
    out = np.zeros((T, H, d))
    for a in range(H):
        g = a // (H // G)
        out[:, a] = softmax_masked((q[:, a] @ k[:, g].T) * m["scale"], seen) @ v[:, g]
    return r(out.reshape(T, H * d)) @ w[p + "o"].T


def short_convolution(x, taps):
    """x [T, C], taps [C, n]: y_t = sum_j taps[:, j] x_{t - (n-1) + j}, zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((n - 1, x.shape[1])), x], axis=0)
    return sum(padded[j:j + T] * taps[:, j] for j in range(n))


def unit_vector(x):
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + 1e-6)


def delta_rule(q, k, v, g, beta):
    """One head: q, k, g [T, d], v [T, dv], beta [T]; returns o [T, dv] and the last state."""
    T, d = q.shape
    S = np.zeros((d, v.shape[1]))
    o = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o, S


def channel_delta(h, w, p, m, eps, r=_id):
    """Gated delta rule with a decay per head and key channel, short convolutions in front of it and
    a gated unit norm behind it."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = r(silu(r(short_convolution(r(h @ w[p + "q"].T), w[p + "q.conv"])))).reshape(T, G, d)
    k = r(silu(r(short_convolution(r(h @ w[p + "k"].T), w[p + "k.conv"])))).reshape(T, G, d)
    v = r(silu(r(short_convolution(r(h @ w[p + "v"].T), w[p + "v.conv"])))).reshape(T, H, dv)
    q = unit_vector(q) * d ** -0.5
    k = unit_vector(k)
    beta = sigmoid(h @ w[p + "b"].T)
    dt = softplus(r(h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, d)
    g = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * dt)
    gate = sigmoid(r(h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for a in range(H):
        kv = a // (H // G)
        o, _S = delta_rule(q[:, kv], k[:, kv], v[:, a], g[:, a], beta[:, a])
        out[:, a] = rms_norm(o, w[p + "norm"], eps) * gate[:, a]
    return r(out.reshape(T, H * dv)) @ w[p + "o"].T


MIXERS = {"latent_attention": latent_attention, "attention": chunked_attention, "channel_delta": channel_delta}


# ---- feed-forward and the per-layer token input ------------------------------------------------
def dense_ffn(h, w, p, r=_id):
    return r(gelu_tanh(r(h @ w[p + "gate"].T)) * r(h @ w[p + "up"].T)) @ w[p + "down"].T


def token_side(x, tokens, w, i, dim, eps, r=_id):
    """What layer i adds for the tokens themselves: a gated slice of a second embedding, projected and normed."""
    e = w["side.embed"][np.asarray(tokens), i * dim:(i + 1) * dim]
    g = r(gelu_tanh(r(r(x) @ w[f"l{i}.side.gate"].T)) * e)
    y = g @ w[f"l{i}.side.proj"].T
    return rms_norm(y, w[f"l{i}.side.norm"], eps)


# ---- the model ---------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], round_fn=_id, layers_out: List = None) -> np.ndarray:
    """Logits [T, vocab] for one sequence from its first token."""
    r = round_fn
    eps = float(cfg["norm"]["eps"])
    side = cfg.get("token_side")
    x = w["embed"][np.asarray(tokens)].astype(np.float64)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = r(rms_norm(x, w[p + "norm1"], eps))
        d = MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps, r)
        if layer.get("mlp") is not None:
            d = d + dense_ffn(h, w, p + "mlp.", r)
        x = x + d
        if side:
            x = x + token_side(x, tokens, w, i, int(side["dim"]), eps, r)
        if layers_out is not None:
            layers_out.append(x.copy())
    return r(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
