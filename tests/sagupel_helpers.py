"""Shared by the Sagupel tests: small configurations of their own, weights drawn so that every mechanism matters (O(1)
activations, biases, sinks, head numbers and a head mix that are far from 0, 1 and the identity, decays from fast to
almost none, sharp attention), model folders."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_sagupel as ps


def retention(heads=3, dim=16, vdim=8, dims=8, base=10000.0, decay=None):
    m = {"decay": list(decay) if decay is not None else [1.0 - 2.0 ** -(3 + 2 * h) for h in range(heads)], "dim": dim,
         "heads": heads, "vdim": vdim}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims}
    return {"type": "retention", "mixer": m}


def attention(heads=4, kv_heads=2, dim=16, size=20, scale=0.3):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": dim}
    if size:
        m["mask"] = {"size": size}
    return {"type": "attention", "mixer": m}


def left(heads=4, kv_heads=2, dim=16, dims=8, base=10000.0, factor=4.0, scale=0.3, softcap=6.0):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": dim}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims}
        if factor:
            m["rot"]["scaling"] = {"factor": factor}
    if softcap:
        m["softcap"] = softcap
    return m


def right(heads=2, kv_heads=1, dim=16, vdim=24, conv=4):
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}


def parallel(left_m=None, right_m=None):
    return {"type": "parallel", "mixer": {"left": left_m or left(), "right": right_m or right()}}


def dense(ff=96, limit=1.25):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(layers, width=64, vocab=96, eps=2e-5, alpha=1.5, taps=4):
    """layers: (mixer entry, mlp entry or None) pairs."""
    out = {"architecture": "Sagupel", "layers": [{**mix, "mlp": mlp} for mix, mlp in layers], "norm": {"eps": eps},
           "vocab": vocab, "width": width}
    if alpha is not None:
        out["postln_alpha"] = alpha
    if taps:
        out["canon"] = {"taps": taps}
    return out


# Sizes that share no value where they could be confused: key/value heads fewer than heads, keys larger than values and
# the other way round, windows that do not divide the page of 64 and one that spans pages, rotations of a part of a head
# and of all of it, two to four taps, a layer without a feed-forward, sizes that are no multiple of 8.
MIXED = config([(retention(heads=3, dim=16, vdim=8, dims=8), dense()),
                (parallel(left(heads=4, kv_heads=2, dim=24, dims=8, factor=4.0), right(heads=2, kv_heads=1, dim=16, vdim=24, conv=4)), dense(ff=40, limit=0.8)),
                (attention(heads=6, kv_heads=2, dim=8, size=20), None),
                (attention(heads=3, kv_heads=3, dim=40, size=70, scale=0.2), dense(ff=72, limit=3.0)),
                (retention(heads=2, dim=24, vdim=40, dims=24, base=500.0, decay=(0.9, 0.999)), dense(ff=24)),
                (parallel(left(heads=6, kv_heads=1, dim=8, dims=2, factor=0, scale=0.6, softcap=2.5),
                          right(heads=3, kv_heads=3, dim=8, vdim=8, conv=2)), None),
                (attention(heads=2, kv_heads=1, dim=12, size=5), dense(ff=56))],
               width=64, vocab=96)
# values that happen to be equal or 1: one head, a window of one position, one tap, no rotation, a constant of 1 on the
# stream, a decay of 1, no cap, no window at all
ONES = config([(retention(heads=1, dim=8, vdim=8, dims=None, decay=(1.0,)), None),
               (parallel(left(heads=1, kv_heads=1, dim=8, dims=None, softcap=0.0), right(heads=1, kv_heads=1, dim=8, vdim=8, conv=1)), dense(ff=16, limit=1.0)),
               (attention(heads=1, kv_heads=1, dim=8, size=1), None),
               (attention(heads=2, kv_heads=2, dim=8, size=0), dense(ff=8))],
              width=16, vocab=37, eps=1e-6, alpha=None, taps=1)


def draw_weights(cfgd, seed=0, sharp=1.0):
    """float64 arrays by tensor name, every value a bfloat16 number, from the configuration alone.  ``sharp`` scales the
    query norms' weights: a sharper softmax shows a key that is seen or not seen."""
    rng = np.random.default_rng(seed)
    D, V = cfgd["width"], cfgd["vocab"]
    taps = (cfgd.get("canon") or {}).get("taps", 0)
    w = {}

    def matrix(*shape):
        return 1.3 * rng.standard_normal(shape) / np.sqrt(shape[-1])

    def norm_weight(n):
        return 1.0 + 0.3 * rng.standard_normal(n)

    w["embed"] = rng.standard_normal((V, D))
    w["embed.norm"], w["final.norm"] = norm_weight(D), norm_weight(D)
    for i, layer in enumerate(cfgd["layers"]):
        px, m = f"l{i}.", layer["mixer"]
        w[px + "norm1"] = norm_weight(D)
        if taps:
            w[px + "canon1"] = 0.5 * rng.standard_normal((D, taps))

        def softmax_attention(p, a):
            H, G, dim = a["heads"], a["kv_heads"], a["dim"]
            w[p + "q"], w[p + "k"], w[p + "o"] = matrix(H * dim, D), matrix(G * dim, D), matrix(D, H * dim)
            w[p + "q.norm"], w[p + "k.norm"] = sharp * norm_weight(dim), norm_weight(dim)

        if layer["type"] == "retention":
            p, H, K, P = px + "mix.", m["heads"], m["dim"], m["vdim"]
            w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"] = matrix(H * K, D), matrix(H * K, D), matrix(H * P, D), matrix(H * P, D)
            w[p + "o"] = matrix(D, H * P)
        elif layer["type"] == "attention":
            softmax_attention(px + "mix.", m)
            w[px + "mix.sink"] = 1.0 + rng.standard_normal(m["heads"])
        else:
            a, r = m["left"], m["right"]
            p, H = px + "mix.left.", a["heads"]
            softmax_attention(p, a)
            w[p + "q.b"], w[p + "k.b"] = 0.4 * rng.standard_normal(H * a["dim"]), 0.4 * rng.standard_normal(a["kv_heads"] * a["dim"])
            w[p + "temp"] = 1.0 + 0.4 * rng.standard_normal(H)
            w[p + "talk"] = np.eye(H) + 0.4 * rng.standard_normal((H, H))
            w[p + "g"] = matrix(H, D)
            p, H, Hk, K, P, c = px + "mix.right.", r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            for name, n in (("q", Hk * K), ("k", Hk * K), ("v", H * P)):
                w[p + name], w[p + name + ".conv"] = matrix(n, D), 0.6 * rng.standard_normal((n, c))
            w[p + "b"], w[p + "a"], w[p + "g"], w[p + "o"] = matrix(H, D), matrix(H, D), matrix(H * P, D), matrix(D, H * P)
            # exp(-exp(A_log) softplus(.)): from a decay of a few tokens to one of hundreds
            w[p + "A_log"], w[p + "dt_bias"] = rng.uniform(-4.0, 0.5, H), rng.uniform(-2.0, 1.0, H)
            w[p + "norm"] = norm_weight(P)
            w[px + "mix.left.out"], w[px + "mix.right.out"] = norm_weight(D), norm_weight(D)
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            w[px + "norm2"] = norm_weight(D)
            w[px + "mlp.gate"], w[px + "mlp.up"], w[px + "mlp.down"] = 2.0 * matrix(ff, D), 2.0 * matrix(ff, D), matrix(D, ff)
    return {k: ps.round_bf16(v) for k, v in w.items()}


def write_folder(path, cfgd, w):
    from questwend_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfgd, f)
    return str(path)
