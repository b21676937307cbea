"""Configuration of the Sagupel design: a decoder whose layers are listed one by one.  The stream is normed AFTER each
sum: ``x <- norm1(alpha x + mixer(x))``, ``x <- norm2(alpha x + feed_forward(x))``, and what the mixer reads first passes
a short causal convolution over time (``canon``).  The mixer is retention (linear attention with a fixed decay per head),
windowed softmax attention with a distance bias and a sink, or a pair that reads the same input: softmax attention
with capped scores, a learned number per head, heads mixed after the softmax and a gate per head, beside the gated delta
rule with one decay per head.  Neither attention has a value projection: a token's value is the raw output of its key projection.

config.json:  ``architecture`` (the design's name), ``vocab``, ``width``, ``norm.eps``, ``postln_alpha``, ``canon.taps``,
``layers``: a list of ``{"type": "retention" | "parallel" | "attention", "mixer": {sizes and constants}, "mlp": {"kind":
"dense", "ff": n, "limit": c} | null}``.  Every size and constant that can differ between two models of the design is
read from there.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..kernels.limits import conv_taps_refusal, shaped_attention_refusal, state_matrix_refusal
from .base import ConfigError, ConfigReader, ModelConfig

ARCHITECTURE = "Sagupel"
MIXER_TYPES = ("retention", "parallel", "attention")


def _sub(r: ConfigReader, key: str, optional: bool = False):
    m = r.mapping(key, None) if optional else r.mapping(key)
    return None if m is None else ConfigReader(m, f"{r.where}: '{key}'")


def _refuse(where: str, refusal):
    if refusal:
        raise ConfigError(f"{where}: {refusal}")


def _read_rotation(r: ConfigReader, dim: int):
    """``rot`` {base, dims} with an optional ``scaling`` {factor}; None where a mixer has no rotation."""
    rot = _sub(r, "rot", optional=True)
    if rot is None:
        return None
    out = {"base": rot.number("base", positive=True), "dims": rot.integer("dims", minimum=0)}
    if out["dims"] % 2 or out["dims"] > dim:
        raise ConfigError(f"{rot.where}: key 'dims' ({out['dims']}) must be even and at most 'dim' ({dim})")
    sc = _sub(rot, "scaling", optional=True)
    if sc is not None:
        out["scaling"] = {"factor": sc.number("factor", positive=True)}
    return out


def _read_heads(r: ConfigReader, grouped: bool = True) -> dict:
    m = {k: r.integer(k, minimum=1) for k in (("dim", "heads", "kv_heads", "vdim") if grouped else ("dim", "heads", "vdim"))}
    if grouped and m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{r.where}: key 'heads' ({m['heads']}) must be a multiple of 'kv_heads' ({m['kv_heads']})")
    return m


def _read_softmax_attention(r: ConfigReader) -> dict:
    """The keys that both softmax attentions of the design share."""
    m = _read_heads(r)
    m["scale"] = r.number("scale", positive=True)
    if m["vdim"] != m["dim"]:
        raise ConfigError(f"{r.where}: key 'vdim' ({m['vdim']}) must equal 'dim' ({m['dim']}): the values are the keys")
    _refuse(f"{r.where}: keys 'dim' and 'vdim'", shaped_attention_refusal(m["dim"], m["vdim"]))
    return m


def _read_mixer(kind: str, r: ConfigReader) -> dict:
    if kind == "retention":
        m = _read_heads(r, grouped=False)
        r.read_keys.add("decay")
        decay = r.data.get("decay")
        if (not isinstance(decay, list) or len(decay) != m["heads"]
                or any(isinstance(d, bool) or not isinstance(d, (int, float)) or not 0.0 <= d <= 1.0 for d in decay)):
            raise ConfigError(f"{r.where}: key 'decay' must list one number in [0, 1] for each of the {m['heads']} heads")
        m["decay"] = [float(d) for d in decay]
        m["rot"] = _read_rotation(r, m["dim"])
        _refuse(f"{r.where}: keys 'dim' and 'vdim'", state_matrix_refusal(m["dim"], m["vdim"]))
        return m
    if kind == "attention":
        m = _read_softmax_attention(r)
        mask = _sub(r, "mask", optional=True)
        m["mask"] = None if mask is None else {"size": mask.integer("size", minimum=1)}
        return m
    left = _read_softmax_attention(_sub(r, "left"))
    lr = ConfigReader(r.data["left"], f"{r.where}: 'left'")
    left["softcap"] = lr.number("softcap", 0.0)
    if left["softcap"] < 0:
        raise ConfigError(f"{lr.where}: key 'softcap' must be >= 0, got {left['softcap']}")
    left["rot"] = _read_rotation(lr, left["dim"])
    rr = _sub(r, "right")
    right = _read_heads(rr)
    right["conv"] = rr.integer("conv", minimum=1)
    _refuse(f"{rr.where}: key 'conv'", conv_taps_refusal(right["conv"]))
    _refuse(f"{rr.where}: keys 'dim' and 'vdim'", state_matrix_refusal(right["dim"], right["vdim"]))
    return {"left": left, "right": right}


def _read_mlp(r: ConfigReader | None):
    if r is None:
        return None
    kind = r.string("kind")
    if kind != "dense":
        raise ConfigError(f"{r.where}: key 'kind' must be 'dense', got {kind!r}")
    return {"kind": "dense", "ff": r.integer("ff", minimum=1), "limit": r.number("limit", positive=True)}


@dataclass(frozen=True)
class SagupelConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float = 1.0
    canon_taps: int = 0                              # 0: the mixers read the stream as it is
    layers: tuple = field(default_factory=tuple)     # dicts: {"type", "mixer": {...}, "mlp": {...} | None}

    architecture = ARCHITECTURE

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "SagupelConfig":
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        alpha = r.number("postln_alpha", 1.0)
        canon = _sub(r, "canon", optional=True)
        taps = 0 if canon is None else canon.integer("taps", minimum=1)
        if taps:
            _refuse(f"{canon.where}: key 'taps'", conv_taps_refusal(taps))
        r.read_keys.add("layers")
        raw = r.data.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError(f"{r.where}: key 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(raw):
            lr = ConfigReader(entry, f"{r.where}: layers[{i}]")
            kind = lr.string("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{lr.where}: key 'type' must be one of {', '.join(MIXER_TYPES)}, got {kind!r}")
            layers.append({"type": kind, "mixer": _read_mixer(kind, _sub(lr, "mixer")), "mlp": _read_mlp(_sub(lr, "mlp", optional=True))})
        return cls(vocab=vocab, width=width, norm_eps=eps, postln_alpha=alpha, canon_taps=taps, layers=tuple(layers))

    def to_dict(self) -> dict:
        import copy
        out = {"architecture": ARCHITECTURE, "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
               "postln_alpha": self.postln_alpha, "vocab": self.vocab, "width": self.width}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        for layer in out["layers"]:                      # keys that stand for "none" are left out again
            m = layer["mixer"]
            for part in ([m["left"]] if layer["type"] == "parallel" else [m]):
                if "rot" in part and part["rot"] is None:
                    del part["rot"]
                if "mask" in part and part["mask"] is None:
                    del part["mask"]
                if "softcap" in part and not part["softcap"]:
                    del part["softcap"]
        return out
