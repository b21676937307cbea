"""The Sagupel design once more, plain and slow: NumPy float64, whole sequences, no cache, no state carried between
calls, one function per mechanism.  It shares no code with the library; the tests compare the engine with it.  A model
is a dict ``cfg`` (the parsed config.json) and a dict ``w`` of float64 arrays by tensor name.

``round16`` rounds where the bfloat16 engine rounds: the operands of the matrix products, the queries, and the cached
keys and values; everything else stays in float64.
"""
from __future__ import annotations

import math

import numpy as np


# ----------------------------------------------------------------------------- small pieces
def round_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


def product(x, W, round16=False):
    """Rows of x times W [out, in] transposed."""
    x = round_bf16(x) if round16 else np.asarray(x, dtype=np.float64)
    return x @ np.asarray(W, dtype=np.float64).T


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


# ----------------------------------------------------------------------------- positions
def rotate_halves(x, positions, dims, base, factor=1.0):
    """x [n, heads, dim]: the first ``dims`` values of every head are turned, value i with value i + dims/2, by the angle
    position * base^(-2i/dims) / factor."""
    if not dims:
        return x
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) / factor for i in range(half)])
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def causal_conv(x, taps_w, plus_input=False):
    """x [n, channels], taps_w [channels, taps]: y_t = sum_j w[:, j] x_(t - taps + 1 + j), zeros before the start."""
    n, taps = x.shape[0], taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, x.shape[1])), x], axis=0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += padded[j:j + n] * taps_w[:, j][None, :]
    return x + y if plus_input else y


# ----------------------------------------------------------------------------- mixers
def retention(h, m, w, px, eps, round16=False):
    """Linear attention with a fixed decay per head."""
    n = h.shape[0]
    H, K, P = m["heads"], m["dim"], m["vdim"]
    q = product(h, w[px + "q"], round16).reshape(n, H, K)
    k = product(h, w[px + "k"], round16).reshape(n, H, K)
    v = product(h, w[px + "v"], round16).reshape(n, H, P)
    pos = np.arange(n)
    rot = m.get("rot") or {}
    q = rotate_halves(q, pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_halves(k, pos, rot.get("dims", 0), rot.get("base", 1.0)) * K ** -0.5
    o = np.zeros((n, H, P))
    for hd in range(H):
        S = np.zeros((K, P))
        for t in range(n):
            S = m["decay"][hd] * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = unit_rms(o, eps).reshape(n, H * P) * silu(product(h, w[px + "g"], round16))
    return product(o, w[px + "o"], round16)


def softmax_attention(h, m, w, px, eps, round16=False, biases=False, rotation=False, softcap=False, temp=False, talk=False,
                      gate=False, slopes=False, sink=False):
    """Grouped-query attention without a value projection: the raw key projections serve as values.  The switches say
    which of the design's two attentions this is."""
    n = h.shape[0]
    H, G, K = m["heads"], m["kv_heads"], m["dim"]
    q = product(h, w[px + "q"], round16)
    k = product(h, w[px + "k"], round16)
    if biases:
        q, k = q + w[px + "q.b"], k + w[px + "k.b"]
    q, k = q.reshape(n, H, K), k.reshape(n, G, K)
    v = k.copy()
    q, k = rms_norm(q, w[px + "q.norm"], eps), rms_norm(k, w[px + "k.norm"], eps)
    if rotation and m.get("rot"):
        rot = m["rot"]
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        pos = np.arange(n)
        q, k = rotate_halves(q, pos, rot["dims"], rot["base"], factor), rotate_halves(k, pos, rot["dims"], rot["base"], factor)
    if round16:
        q, k, v = round_bf16(q), round_bf16(k), round_bf16(v)
    window = (m.get("mask") or {}).get("size", 0)
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    seen = j <= i
    if window:
        seen &= i - j < window
    weights = np.zeros((H, n, n))
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd // (H // G)].T) * m["scale"]
        if temp:
            s = s * w[px + "temp"][hd]
        if softcap and m.get("softcap"):
            s = m["softcap"] * np.tanh(s / m["softcap"])
        if slopes:
            s = s - 2.0 ** (-8.0 * (hd + 1) / H) * (i - j)
        s = np.where(seen, s, -np.inf)
        top = s.max(axis=-1, keepdims=True)
        if sink:
            top = np.maximum(top, w[px + "sink"][hd])
        e = np.exp(s - top)
        total = e.sum(axis=-1, keepdims=True)
        if sink:
            total = total + np.exp(w[px + "sink"][hd] - top)
        weights[hd] = e / total
    if talk:
        weights = np.einsum("hg,gij->hij", w[px + "talk"], weights)
    o = np.stack([weights[hd] @ v[:, hd // (H // G)] for hd in range(H)], axis=1)        # [n, H, K]
    if gate:
        o = o * sigmoid(product(h, w[px + "g"], round16))[:, :, None]
    return product(o.reshape(n, H * K), w[px + "o"], round16)


def gated_delta(h, m, w, px, eps, round16=False):
    """The gated delta rule with one decay per head."""
    n = h.shape[0]
    H, Hk, K, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    parts = []
    for name in ("q", "k", "v"):
        parts.append(silu(causal_conv(product(h, w[px + name], round16), w[px + name + ".conv"])))
    q, k, v = parts[0].reshape(n, Hk, K), parts[1].reshape(n, Hk, K), parts[2].reshape(n, H, P)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * K ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(product(h, w[px + "b"], round16))
    g = np.exp(-np.exp(w[px + "A_log"]) * softplus(product(h, w[px + "a"], round16) + w[px + "dt_bias"]))
    o = np.zeros((n, H, P))
    for hd in range(H):
        kh = hd // (H // Hk)
        S = np.zeros((K, P))
        for t in range(n):
            S = g[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + np.outer(k[t, kh], u)
            o[t, hd] = S.T @ q[t, kh]
    o = rms_norm(o, w[px + "norm"], eps).reshape(n, H * P) * silu(product(h, w[px + "g"], round16))
    return product(o, w[px + "o"], round16)


def parallel(h, m, w, px, eps, round16=False):
    left = softmax_attention(h, m["left"], w, px + "left.", eps, round16, biases=True, rotation=True, softcap=True, temp=True,
                             talk=True, gate=True)
    right = gated_delta(h, m["right"], w, px + "right.", eps, round16)
    return 0.5 * (rms_norm(left, w[px + "left.out"], eps) + rms_norm(right, w[px + "right.out"], eps))


def window_attention(h, m, w, px, eps, round16=False):
    return softmax_attention(h, m, w, px, eps, round16, slopes=True, sink=True)


MIXERS = {"retention": retention, "parallel": parallel, "attention": window_attention}


# ----------------------------------------------------------------------------- feed-forward
def feed_forward(x, mlp, w, px, round16=False):
    limit = mlp["limit"]
    g = np.minimum(product(x, w[px + "gate"], round16), limit)
    u = np.clip(product(x, w[px + "up"], round16), -limit, limit)
    return product(g * sigmoid(1.702 * g) * (u + 1.0), w[px + "down"], round16)


# ----------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, round16=False, taps=None):
    """Logits [n, vocab] of one sequence; ``taps``, a list, receives the stream after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg.get("postln_alpha", 1.0)
    x = rms_norm(w["embed"][np.asarray(tokens)], w["embed.norm"], eps)
    for i, layer in enumerate(cfg["layers"]):
        px = f"l{i}."
        h = causal_conv(x, w[px + "canon1"], plus_input=True) if cfg.get("canon") else x
        x = rms_norm(alpha * x + MIXERS[layer["type"]](h, layer["mixer"], w, px + "mix.", eps, round16), w[px + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = rms_norm(alpha * x + feed_forward(x, layer["mlp"], w, px + "mlp.", round16), w[px + "norm2"], eps)
        if taps is not None:
            taps.append(x.copy())
    return product(rms_norm(x, w["final.norm"], eps), w["embed"], round16)
