"""Shared by the Punolix tests: small configurations of their own, weights drawn so that every mechanism matters
(O(1) activations, biases and loop vectors that are not zero, a lambda far from its constant, decays from fast to almost
none, sharp attention), model folders."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_punolix as pp


def attention(heads=4, kv_heads=2, dim=16, vdim=24, dims=8, base=10000.0, scale=0.3, softcap=6.0, diff=0.25):
    m = {"diff": diff, "dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": {"base": base, "dims": dims}, "scale": scale,
         "vdim": vdim}
    if softcap:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def left(heads=4, kv_heads=2, dim=16, vdim=16, dims=8, base=10000.0, scale=0.3, conv=3, size=20, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "vdim": vdim}
    if conv:
        m["conv"] = conv
    if size:
        m["mask"] = {"size": size}
    return m


def right(heads=2, dim=16, vdim=24, tau=8.0):
    return {"dim": dim, "heads": heads, "tau": tau, "vdim": vdim}


def parallel(left_m=None, right_m=None, left_scale=1.3, right_scale=0.6):
    return {"type": "parallel", "mixer": {"left": left_m or left(), "right": right_m or right(), "left_scale": left_scale,
                                          "right_scale": right_scale}}


def dense(ff=96):
    return {"kind": "dense", "ff": ff}


def config(layers, width=64, vocab=96, eps=1e-5, loop=None, embedding_scale=3.0, residual_mult=0.6):
    """layers: (mixer entry, mlp entry or None) pairs."""
    out = {"architecture": "Punolix", "layers": [{**mix, "mlp": mlp} for mix, mlp in layers], "norm": {"eps": eps},
           "vocab": vocab, "width": width}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if embedding_scale is not None:
        out["embedding"] = {"scale": embedding_scale}
    if residual_mult is not None:
        out["residual_mult"] = residual_mult
    return out


# Sizes that share no value where they could be confused: key/value heads fewer than heads, keys larger than values and
# the other way round, a chunk that does not divide the page of 64 and one that spans pages, rotations of a part of a
# map and of all of it, frequencies scaled so that all three bands occur, two to four taps, a looped run that starts
# after the first layer, a layer without a feed-forward.
MIXED = config([(attention(heads=4, kv_heads=2, dim=16, vdim=24, dims=8), dense()),
                (parallel(left(heads=4, kv_heads=2, dim=24, vdim=16, dims=8, conv=3, size=20, scaling=(4.0, 1.0, 4.0, 64)),
                          right(heads=2, dim=16, vdim=24, tau=8.0)), dense(ff=40)),
                (attention(heads=3, kv_heads=3, dim=8, vdim=40, dims=8, base=500.0, softcap=2.5, diff=0.4), None),
                (parallel(left(heads=6, kv_heads=1, dim=8, vdim=8, dims=2, conv=4, size=70, scale=0.6),
                          right(heads=3, dim=8, vdim=8, tau=3.0), left_scale=0.7, right_scale=1.1), dense(ff=72)),
                (attention(heads=2, kv_heads=1, dim=32, vdim=8, dims=32, softcap=0.0, diff=0.1), dense(ff=24))],
               width=64, vocab=96, loop=(1, 4, 3))
# values that happen to be equal or 1: one head, a chunk of one position, two taps, no rotation, a loop of one pass, no
# scale on the embedding, a residual factor of 1, scales of 1, a decay exponent of 1
ONES = config([(parallel(left(heads=1, kv_heads=1, dim=8, vdim=8, dims=0, conv=2, size=1),
                         right(heads=1, dim=8, vdim=8, tau=1.0), left_scale=1.0, right_scale=1.0), None),
               (attention(heads=1, kv_heads=1, dim=8, vdim=8, dims=0, softcap=0.0, diff=0.0), dense(ff=16)),
               (parallel(left(heads=2, kv_heads=2, dim=8, vdim=8, dims=8, conv=0, size=0), right(heads=2, dim=8, vdim=8, tau=2.0)), None)],
              width=16, vocab=37, eps=1e-6, loop=(0, 2, 1), embedding_scale=None, residual_mult=None)
DECAY_RANK = 5


def draw_weights(cfgd, seed=0, slow_decay=False, sharp=1.0, rank=DECAY_RANK):
    """float64 arrays by tensor name, every value a bfloat16 number, from the configuration alone.  ``sharp`` scales the
    query projections and norm weights: a sharper softmax shows a key that is seen or not seen."""
    rng = np.random.default_rng(seed)
    D, V = cfgd["width"], cfgd["vocab"]
    escale = cfgd.get("embedding", {}).get("scale", 1.0)
    w = {}

    def matrix(*shape):
        return 1.3 * rng.standard_normal(shape) / np.sqrt(shape[-1])

    def norm_weight(n):
        return 1.0 + 0.3 * rng.standard_normal(n)

    w["embed"] = rng.standard_normal((V, D)) / escale
    w["final.norm"] = norm_weight(D)
    w["head"] = matrix(V, D)
    if cfgd.get("loop"):
        w["loop.step"] = 0.7 * rng.standard_normal((cfgd["loop"]["times"], D))
    for i, layer in enumerate(cfgd["layers"]):
        px, m = f"l{i}.", layer["mixer"]
        w[px + "norm1"] = norm_weight(D)

        def softmax_attention(p, a, maps):
            H, G, dim, vdim = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            w[p + "q"], w[p + "k"], w[p + "v"] = sharp * matrix(H * maps * dim, D), matrix(G * maps * dim, D), matrix(G * vdim, D)
            w[p + "o"] = matrix(D, H * vdim)
            for name, n in (("q", H * maps * dim), ("k", G * maps * dim), ("v", G * vdim)):
                w[p + name + ".b"] = 0.4 * rng.standard_normal(n)
                if a.get("conv"):
                    w[p + name + ".conv"] = 0.6 * rng.standard_normal((n, a["conv"]))

        if layer["type"] == "attention":
            softmax_attention(px + "mix.", m, 2)
            for name in ("lq1", "lk1", "lq2", "lk2"):                       # lambda = e^a - e^b + diff with a, b of order 1/2
                w[px + "mix." + name] = 0.9 * rng.standard_normal(m["dim"]) / m["dim"] ** 0.25
        else:
            a, r = m["left"], m["right"]
            softmax_attention(px + "mix.left.", a, 1)
            w[px + "mix.left.o.b"] = 0.4 * rng.standard_normal(D)
            w[px + "mix.left.q.norm"], w[px + "mix.left.k.norm"] = sharp * norm_weight(a["dim"]), norm_weight(a["dim"])
            p, H, dim, vdim = px + "mix.right.", r["heads"], r["dim"], r["vdim"]
            w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"] = matrix(H * dim, D), matrix(H * dim, D), matrix(H * vdim, D), matrix(H * vdim, D)
            w[p + "o"], w[p + "norm"] = matrix(D, H * vdim), norm_weight(vdim)
            w[p + "a1"], w[p + "a2"] = matrix(rank, D), 2.0 * matrix(H * dim, rank)
            # sigmoid(z)^(1/tau): with z around 6 the state keeps hundreds of tokens, around 0 a few
            w[p + "a2.b"] = rng.uniform(5.0, 8.0, H * dim) if slow_decay else rng.uniform(-2.0, 5.0, H * dim)
        if layer["mlp"]:
            ff = layer["mlp"]["ff"]
            w[px + "mlp.gate"], w[px + "mlp.up"], w[px + "mlp.down"] = matrix(ff, D), matrix(ff, D), matrix(D, ff)
    return {k: pp.round_bf16(v) for k, v in w.items()}


def write_folder(path, cfgd, w):
    from questwend_b200.weights import write_safetensors
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16) for k, v in w.items()})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfgd, f)
    return str(path)
