"""Punolix: configuration -> plan.

Every layer is ``x = norm1(h); h += m * (mixer(x) + feed_forward(x))`` with an RMS norm and one constant m for the
model; the mixer is differential attention (two score maps per head, soft-capped scores, a rotation of neighbouring
pairs) or two mixers side by side: attention inside chunks of positions behind a short convolution of q, k and v (q/k
norm, a rotation of half-apart pairs whose frequencies may be scaled by wavelength) and gated linear attention; the
feed-forward is dense and gated with the tanh form of GELU, or absent.  A run of layers may be looped: the schedule names
those layers several times, each run with a cache and state of its own, and every pass opens with a step that adds the
embedding output again (all passes but the first) and the pass's row of ``loop.step``.  Tensors: ``embed``,
``loop.step``, ``l<i>.norm1``, ``l<i>.mix.*`` (``.left.*`` / ``.right.*`` for the pair), ``l<i>.mlp.*``, ``final.norm``,
``head``.  The rank of the linear attention's decay projection is not in a config.json; the tensors' shapes give it.
"""
from __future__ import annotations

from ..config.punolix import ARCHITECTURE, PunolixConfig
from ..config.registry import register_architecture
from ..engine.plan import LayerSpec, ModelPlan, Run
from ..parts.base import PartSpec

DEFAULT_DECAY_RANK = 16     # for a configuration that was not read beside its weights (random weights)


def _rotation(rot: dict):
    if not rot["dims"]:
        return None
    return PartSpec("rotary_wavelength", {"theta": rot["base"], "rotary_dim": rot["dims"], **dict(rot.get("scaling") or {})})


def _softmax_attention(m: dict, width: int, eps: float, **more):
    return PartSpec("score_maps_attention",
                    {"hidden_size": width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                     "value_dim": m["vdim"], "biases": True, "conv": m["conv"], "norm_eps": eps, "scale": m["scale"],
                     "softcap": m["softcap"], "chunk": m["mask"]["size"] if m["mask"] else 0, **more})


def _mixer(kind: str, m: dict, width: int, eps: float):
    """(mixer spec, position spec(s) or None)."""
    if kind == "attention":
        return _softmax_attention(m, width, eps, maps=2, diff=m["diff"], layout="interleaved"), _rotation(m["rot"])
    left, right = m["left"], m["right"]
    gla = PartSpec("gated_linear_attention",
                   {"hidden_size": width, "heads": right["heads"], "key_dim": right["dim"], "vdim": right["vdim"],
                    "decay_rank": right.get("rank", DEFAULT_DECAY_RANK), "tau": right["tau"], "norm_eps": eps})
    pair = PartSpec("side_by_side", {"branches": (
        {"name": "left", "spec": _softmax_attention(left, width, eps, maps=1, qk_norm=True, out_bias=True, layout="halves"),
         "scale": m["left_scale"]},
        {"name": "right", "spec": gla, "scale": m["right_scale"]})})
    return pair, (_rotation(left["rot"]), None)


def _feed_forward(mlp, width: int):
    if mlp is None:
        return None
    return PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": mlp["ff"], "activation": "gelu_tanh",
                                  "names": {"gate": "gate", "up": "up", "down": "down"}})


def punolix_plan(cfg: PunolixConfig) -> ModelPlan:
    D, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rms", {"dim": D, "eps": eps})
    layers = []
    for i, layer in enumerate(cfg.layers):
        mixer, position = _mixer(layer["type"], layer["mixer"], D, eps)
        layers.append(LayerSpec(block=PartSpec("parallel_residual", {"norm": "norm1", "mixer_prefix": "mix", "ffn_prefix": "mlp",
                                                                     "residual_mult": cfg.residual_mult}, prefix=f"l{i}."),
                                mixer=mixer, feed_forward=_feed_forward(layer["mlp"], D), norm=norm, position=position))
    embed = {"vocab_size": cfg.vocab, "hidden_size": D, "name": "embed", "scale": cfg.embedding_scale}
    times = cfg.loop[2] if cfg.loop is not None else 0
    schedule = []
    for layer, opens in cfg.passes():
        before = None
        if opens is not None:
            before = PartSpec("reinject_embedding", {**embed, "add_embedding": opens > 0, "vector": "loop.step", "rows": times,
                                                     "row": opens})
        schedule.append(Run(layer, before=before))
    return ModelPlan(
        architecture=ARCHITECTURE, hidden_size=D, vocab_size=cfg.vocab,
        embedding=PartSpec("token", embed), layers=layers, schedule=schedule,
        final_norm=PartSpec("rms", {"dim": D, "eps": eps, "name": "final.norm"}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "hidden_size": D, "tied": False, "name": "head", "tied_to": "embed"}),
        stop_token_ids=(), max_position=None)


register_architecture(ARCHITECTURE, PunolixConfig, punolix_plan, replace=True)
