"""The Punolix design once more, plain and slow: NumPy float64, whole sequences, no cache, no state carried between
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x over its root mean square along the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def softmax(s):
    """Along the last axis; -inf entries get weight 0."""
    e = np.exp(s - np.max(s, axis=-1, keepdims=True))
    return e / np.sum(e, axis=-1, keepdims=True)


# ----------------------------------------------------------------------------- rotation
def frequencies(base, dims, scaling=None):
    """Angle per position of pair i: base^(-2i/dims); with ``scaling`` {factor, low, high, original} long wavelengths
    are slowed by ``factor``, short ones kept, and those between blended."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return np.array(out)


def rotate(x, positions, freqs, dims, layout):
    """x [T, ..., n]: the first ``dims`` values of the last axis turn by position * freqs; "interleaved" pairs value 2i
    with 2i + 1, "halves" pairs value i with i + dims / 2."""
    if not dims:
        return x
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = np.cos(angle).reshape(shape), np.sin(angle).reshape(shape)
    out = x.copy()
    if layout == "interleaved":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = a * c - b * s, b * c + a * s
    return out


# ----------------------------------------------------------------------------- mechanisms
def short_convolution(u, taps_w):
    """u [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u])
    return sum(padded[j:j + T] * taps_w[:, j][None, :] for j in range(taps))


def visible(T, chunk=0):
    """[T, T] booleans: key j is seen from position i when j <= i and, with chunks, both lie in the same chunk."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    ok = j <= i
    if chunk:
        ok &= (i // chunk) == (j // chunk)
    return ok


def attention_map(q, k, v, scale, mask, softcap=0.0):
    """One softmax attention: q [T, n], k [T, n], v [T, m]."""
    s = q @ k.T * scale
    if softcap:
        s = softcap * np.tanh(s / softcap)
    return softmax(np.where(mask, s, -np.inf)) @ v


def differential_attention(h, w, px, m, eps, round16=False):
    """Two score maps per head over the same values; their outputs are subtracted, normed and scaled."""
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = np.arange(T)
    q = (product(h, w[px + "q"], round16) + w[px + "q.b"]).reshape(T, H, 2, n)
    k = (product(h, w[px + "k"], round16) + w[px + "k.b"]).reshape(T, G, 2, n)
    v = (product(h, w[px + "v"], round16) + w[px + "v.b"]).reshape(T, G, nv)
    f = frequencies(m["rot"]["base"], m["rot"]["dims"])
    q, k = rotate(q, pos, f, m["rot"]["dims"], "interleaved"), rotate(k, pos, f, m["rot"]["dims"], "interleaved")
    if round16:
        q, k, v = round_bf16(q), round_bf16(k), round_bf16(v)
    lam = math.exp(float(w[px + "lq1"] @ w[px + "lk1"])) - math.exp(float(w[px + "lq2"] @ w[px + "lk2"])) + m["diff"]
    mask = visible(T, (m.get("mask") or {}).get("size", 0))
    heads = []
    for head in range(H):
        g = head // (H // G)
        a1, a2 = (attention_map(q[:, head, i], k[:, g, i], v[:, g], m["scale"], mask, m.get("softcap", 0.0)) for i in (0, 1))
        heads.append(unit_rms(a1 - lam * a2, eps) * (1.0 - m["diff"]))
    return product(np.concatenate(heads, axis=1), w[px + "o"], round16)


def chunked_attention(h, w, px, m, eps, round16=False):
    """Softmax attention inside chunks of positions, behind a short convolution, a q/k norm and a rotation."""
    H, G, n, nv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    pos = np.arange(T)
    proj = {}
    for name in "qkv":
        u = product(h, w[px + name], round16) + w[px + name + ".b"]
        proj[name] = short_convolution(u, w[px + name + ".conv"]) if m.get("conv") else u
    q = rms_norm(proj["q"].reshape(T, H, n), w[px + "q.norm"], eps)
    k = rms_norm(proj["k"].reshape(T, G, n), w[px + "k.norm"], eps)
    v = proj["v"].reshape(T, G, nv)
    f = frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    q, k = rotate(q, pos, f, m["rot"]["dims"], "halves"), rotate(k, pos, f, m["rot"]["dims"], "halves")
    if round16:
        q, k, v = round_bf16(q), round_bf16(k), round_bf16(v)
    mask = visible(T, (m.get("mask") or {}).get("size", 0))
    heads = [attention_map(q[:, head], k[:, head // (H // G)], v[:, head // (H // G)], m["scale"], mask, m.get("softcap", 0.0))
             for head in range(H)]
    return product(np.concatenate(heads, axis=1), w[px + "o"], round16) + w[px + "o.b"]


def gated_linear_attention(h, w, px, m, eps, round16=False):
    """Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T from S = 0, o_t = S_t^T q_t; normed, gated, projected."""
    H, n, nv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = product(h, w[px + "q"], round16).reshape(T, H, n) * n ** -0.5
    k = product(h, w[px + "k"], round16).reshape(T, H, n)
    v = product(h, w[px + "v"], round16).reshape(T, H, nv)
    z = product(product(h, w[px + "a1"], round16), w[px + "a2"], round16) + w[px + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, n)
    S = np.zeros((H, n, nv))
    o = np.zeros((T, H, nv))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hnv,hn->hv", S, q[t])
    o = rms_norm(o, w[px + "norm"], eps).reshape(T, H * nv)
    return product(o * silu(product(h, w[px + "g"], round16)), w[px + "o"], round16)


def side_by_side(h, w, px, m, eps, round16=False):
    return (m["left_scale"] * chunked_attention(h, w, px + "left.", m["left"], eps, round16)
            + m["right_scale"] * gated_linear_attention(h, w, px + "right.", m["right"], eps, round16))


def gated_feed_forward(h, w, px, round16=False):
    return product(gelu_tanh(product(h, w[px + "gate"], round16)) * product(h, w[px + "up"], round16), w[px + "down"], round16)


def mixer(kind, h, w, px, m, eps, round16=False):
    return (differential_attention if kind == "attention" else side_by_side)(h, w, px, m, eps, round16)


# ----------------------------------------------------------------------------- the model
def runs(cfg):
    """(layer, pass that the run opens or None) in the order of execution."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(tokens, w, cfg, round16=False, layers_out=None):
    """Logits [T, vocab] of one whole sequence."""
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x0 = np.asarray(w["embed"], dtype=np.float64)[np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    x = x0.copy()
    for i, opens in runs(cfg):
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + w["loop.step"][opens]
        layer, px = cfg["layers"][i], f"l{i}."
        h = rms_norm(x, w[px + "norm1"], eps)
        y = mixer(layer["type"], h, w, px + "mix.", layer["mixer"], eps, round16)
        if layer.get("mlp"):
            y = y + gated_feed_forward(h, w, px + "mlp.", round16)
        x = x + mult * y
        if layers_out is not None:
            layers_out.append(x.copy())
    return product(rms_norm(x, w["final.norm"], eps), w["head"], round16)
