"""Sagupel: configuration -> plan.

Every layer is ``x <- norm1(alpha x + mixer(x))``, then ``x <- norm2(alpha x + feed_forward(x))`` with RMS norms: the
norm comes after the sum, and the sublayers read the normed stream itself.  What the mixer reads first passes
``x + conv(x)``, a short causal convolution over time on every channel.  The mixer is retention (linear attention with
a fixed decay per head, rotated q and k), softmax attention over a sliding window with a bias that grows with distance
and a learned sink per head, or two mixers side by side, each output RMS-normed and the two averaged: softmax attention
with biased projections, rotated q and k with linearly scaled positions, capped scores, a learned number per head, heads
mixed after the softmax and a gate per head; and the gated delta rule with one decay per head.  Neither softmax
attention has a value projection: a token's value is the raw output of its key projection.  The feed-forward is dense with a clamped gate.  The embedding output is
RMS-normed; the output head is the embedding table.  Tensors: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.canon1``, ``l<i>.mix.*`` (``.left.*`` / ``.right.*`` for the pair), ``l<i>.mlp.*``, ``final.norm``.
What the design fixes (which sublayers have biases, the pairing of the rotation, the slopes' base, the activations) stands
here as parameters of the parts.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sagupel import ARCHITECTURE, SagupelConfig
from ..engine.plan import LayerSpec, ModelPlan, Run
from ..parts.base import PartSpec

SLOPE_BASE = 8.0            # the distance bias of head h of H has the slope 2^(-8 (h + 1) / H)


def _rotation(rot):
    if not rot or not rot["dims"]:
        return None
    return PartSpec("rotary_neox", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                    "linear_factor": (rot.get("scaling") or {}).get("factor", 1.0)})


def _attention(m: dict, width: int, eps: float, **more):
    return PartSpec("shaped_score_attention",
                    {"hidden_size": width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                     "value_dim": m["vdim"], "values_from_keys": True, "qk_norm": True, "norm_eps": eps, "scale": m["scale"],
                     "layout": "halves", **more})


def _mixer(kind: str, m: dict, width: int, eps: float):
    """(mixer spec, position spec(s) or None)."""
    if kind == "retention":
        return PartSpec("retention", {"hidden_size": width, "heads": m["heads"], "key_dim": m["dim"], "vdim": m["vdim"],
                                      "decay": tuple(m["decay"]), "norm_eps": eps}), _rotation(m["rot"])
    if kind == "attention":
        return _attention(m, width, eps, slope_base=SLOPE_BASE, window=m["mask"]["size"] if m["mask"] else 0, sink=True), None
    left, right = m["left"], m["right"]
    delta = PartSpec("gated_delta_headwise",
                     {"hidden_size": width, "heads": right["heads"], "key_heads": right["kv_heads"], "key_dim": right["dim"],
                      "vdim": right["vdim"], "conv": right["conv"], "norm_eps": eps})
    pair = PartSpec("side_by_side", {"branches": (
        {"name": "left", "spec": _attention(left, width, eps, biases=True, head_temperature=True, softcap=left["softcap"],
                                            head_mix=True, head_gate=True),
         "scale": 0.5, "norm": {"name": "left.out", "dim": width, "eps": eps}},
        {"name": "right", "spec": delta, "scale": 0.5, "norm": {"name": "right.out", "dim": width, "eps": eps}})})
    return pair, (_rotation(left["rot"]), None)


def _feed_forward(mlp, width: int):
    if mlp is None:
        return None
    return PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": mlp["ff"], "activation": "clamped_swish",
                                  "limit": mlp["limit"], "names": {"gate": "gate", "up": "up", "down": "down"}})


def sagupel_plan(cfg: SagupelConfig) -> ModelPlan:
    D, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms", {"dim": D, "eps": eps})
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer, position = _mixer(layer["type"], layer["mixer"], D, eps)
        if cfg.canon_taps:
            mixer = PartSpec("input_conv", {"inner": mixer, "channels": D, "taps": cfg.canon_taps, "weight": f"l{i}.canon1"})
        layers.append(LayerSpec(block=PartSpec("post_norm", {"mixer_norm": "norm1", "ffn_norm": "norm2", "mixer_prefix": "mix",
                                                             "ffn_prefix": "mlp", "alpha": cfg.postln_alpha}, prefix=f"l{i}."),
                                mixer=mixer, feed_forward=_feed_forward(layer["mlp"], D), norm=norm, position=position))
    return ModelPlan(
        architecture=ARCHITECTURE, hidden_size=D, vocab_size=cfg.vocab,
        embedding=PartSpec("token", {"vocab_size": cfg.vocab, "hidden_size": D, "name": "embed", "norm": "embed.norm",
                                     "norm_eps": eps}),
        layers=layers, schedule=[Run(i) for i in range(len(layers))],
        final_norm=PartSpec("rms", {"dim": D, "eps": eps, "name": "final.norm"}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "hidden_size": D, "tied": True, "name": "head", "tied_to": "embed"}),
        stop_token_ids=(), max_position=None)


register_architecture(ARCHITECTURE, SagupelConfig, sagupel_plan, replace=True)
