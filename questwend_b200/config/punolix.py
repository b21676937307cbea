"""Configuration of the Punolix design: a decoder whose layers are listed one by one.  A layer norms the stream once and
feeds the result to its mixer and to its feed-forward side by side; their sum, times ``residual_mult``, goes onto the
stream.  The mixer is differential attention (two score maps per head over the same values) or a pair of mixers that
read the same input: chunked attention behind a short convolution, and gated linear attention.  A run of layers may be
looped; every pass starts from the stream plus the embedding output plus a learned vector of its own.

config.json:  ``architecture`` (the design's name), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``residual_mult``, ``layers``: a list of ``{"type": "attention" | "parallel", "mixer": {sizes}, "mlp": {"kind": "dense",
"ff": n} | null}``, and optionally ``loop`` {start, stop, times}.  Every size and constant that can differ between two
models of the design is read from there; the rank of the linear attention's decay projection is the row count of its
first matrix.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..kernels.limits import conv_taps_refusal, maps_attention_refusal, state_matrix_refusal
from .base import ConfigError, ConfigReader, ModelConfig

ARCHITECTURE = "Punolix"
MIXER_TYPES = ("attention", "parallel")
DECAY_RANK_TENSOR = "a1"        # the decay's low rank is the row count of '<layer>.mix.right.a1'


def _sub(r: ConfigReader, key: str, optional: bool = False):
    m = r.mapping(key, None) if optional else r.mapping(key)
    return None if m is None else ConfigReader(m, f"{r.where}: '{key}'")


def _refuse(where: str, refusal):
    if refusal:
        raise ConfigError(f"{where}: {refusal}")


def _read_rotation(r: ConfigReader, dim: int) -> dict:
    rot = _sub(r, "rot")
    out = {"base": rot.number("base", positive=True), "dims": rot.integer("dims", minimum=0)}
    if out["dims"] % 2 or out["dims"] > dim:
        raise ConfigError(f"{rot.where}: key 'dims' ({out['dims']}) must be even and at most 'dim' ({dim})")
    if not out["base"] > 1:
        raise ConfigError(f"{rot.where}: key 'base' must be > 1, got {out['base']}")
    sc = _sub(rot, "scaling", optional=True)
    if sc is not None:
        out["scaling"] = {k: sc.number(k, positive=True) for k in ("factor", "low", "high", "original")}
        if not out["scaling"]["high"] > out["scaling"]["low"]:
            raise ConfigError(f"{sc.where}: key 'high' must be larger than 'low'")
    return out


def _read_softmax_attention(r: ConfigReader, maps: int) -> dict:
    """The keys that both softmax attentions of the design share; ``maps`` score maps per head."""
    w = r.where
    m = {k: r.integer(k, minimum=1) for k in ("dim", "heads", "kv_heads", "vdim")}
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{w}: key 'heads' ({m['heads']}) must be a multiple of 'kv_heads' ({m['kv_heads']})")
    m["scale"] = r.number("scale", positive=True)
    m["softcap"] = r.number("softcap", 0.0)
    if m["softcap"] < 0:
        raise ConfigError(f"{w}: key 'softcap' must be >= 0, got {m['softcap']}")
    m["conv"] = r.integer("conv", 0, minimum=0)
    if m["conv"]:
        _refuse(f"{w}: key 'conv'", conv_taps_refusal(m["conv"]))
    mask = _sub(r, "mask", optional=True)
    m["mask"] = None if mask is None else {"size": mask.integer("size", minimum=1)}
    m["rot"] = _read_rotation(r, m["dim"])
    _refuse(f"{w}: keys 'dim' and 'vdim'", maps_attention_refusal(maps, m["dim"], m["vdim"]))
    return m


def _read_mixer(kind: str, r: ConfigReader) -> dict:
    if kind == "attention":
        m = _read_softmax_attention(r, 2)
        m["diff"] = r.number("diff")
        if not 0.0 <= m["diff"] < 1.0:
            raise ConfigError(f"{r.where}: key 'diff' must lie in [0, 1), got {m['diff']}")
        return m
    left = _read_softmax_attention(_sub(r, "left"), 1)
    rr = _sub(r, "right")
    right = {k: rr.integer(k, minimum=1) for k in ("dim", "heads", "vdim")}
    right["tau"] = rr.number("tau", positive=True)
    if rr.has("rank"):
        right["rank"] = rr.integer("rank", minimum=1)
    _refuse(f"{rr.where}: keys 'dim' and 'vdim'", state_matrix_refusal(right["dim"], right["vdim"]))
    return {"left": left, "right": right, "left_scale": r.number("left_scale", 1.0), "right_scale": r.number("right_scale", 1.0)}


def _read_mlp(r: ConfigReader | None):
    if r is None:
        return None
    kind = r.string("kind")
    if kind != "dense":
        raise ConfigError(f"{r.where}: key 'kind' must be 'dense', got {kind!r}")
    return {"kind": "dense", "ff": r.integer("ff", minimum=1)}


@dataclass(frozen=True)
class PunolixConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    layers: tuple = field(default_factory=tuple)     # dicts: {"type", "mixer": {...}, "mlp": {...} | None}
    loop: tuple | None = None                        # (start, stop, times)

    architecture = ARCHITECTURE

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "PunolixConfig":
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        emb = _sub(r, "embedding", optional=True)
        emb_scale = emb.number("scale", 1.0) if emb is not None else 1.0
        mult = r.number("residual_mult", 1.0)
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
        loop = None
        lp = _sub(r, "loop", optional=True)
        if lp is not None:
            loop = (lp.integer("start", minimum=0), lp.integer("stop", minimum=0), lp.integer("times", minimum=1))
            if not loop[0] < loop[1] <= len(layers):
                raise ConfigError(f"{lp.where}: layers {loop[0]} .. {loop[1]} - 1 do not lie within the {len(layers)} layers")
        return cls(vocab=vocab, width=width, norm_eps=eps, embedding_scale=emb_scale, residual_mult=mult,
                   layers=tuple(layers), loop=loop)

    def with_tensor_shapes(self, shapes) -> "PunolixConfig":
        """The rank of the linear attention's decay projection is the row count of ``l<i>.mix.right.a1``."""
        import copy
        import dataclasses
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            if layer["type"] == "parallel":
                name = f"l{i}.mix.right.{DECAY_RANK_TENSOR}"
                if "rank" not in layer["mixer"]["right"] and name in shapes and len(shapes[name]) == 2:
                    layer["mixer"]["right"]["rank"] = int(shapes[name][0])
        return dataclasses.replace(self, layers=tuple(layers))

    def passes(self) -> list[tuple]:
        """The layers in the order they run, as (layer, pass that this run opens or None): the looped run repeated, the
        rest once."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        out = [(i, None) for i in range(start)]
        for t in range(times):
            out += [(i, t if i == start else None) for i in range(start, stop)]
        return out + [(i, None) for i in range(stop, n)]

    def to_dict(self) -> dict:
        import copy
        out = {"architecture": ARCHITECTURE, "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width, "embedding": {"scale": self.embedding_scale},
               "residual_mult": self.residual_mult}
        for layer in out["layers"]:                      # keys that stand for "none" are left out again
            for m in ([layer["mixer"]] if layer["type"] == "attention" else [layer["mixer"]["left"]]):
                if not m["conv"]:
                    del m["conv"]
                if not m["softcap"]:
                    del m["softcap"]
                if m["mask"] is None:
                    del m["mask"]
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out
