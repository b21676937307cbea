"""Token embedding (a row gather, no scaling; core/runtime.cpp:1001) and the output head
(logits = x W^T with the embedding table as W when the head is tied; core/runtime.cpp:1093-1096)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.manifest import MATRIX, NORM_WEIGHT, VECTOR, TensorSpec
from .base import Part, StreamStep
from .linear import kernel_modules as linear_modules, linear
from .registry import register_embedding, register_head, register_stream_step


class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, name, scale (the rows are multiplied by it; default 1), norm (the tensor name of
    an RMS norm's weight that the rows pass right after the gather; default none) with norm_eps."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.name = self.prefix + spec.params.get("name", "embed_tokens.weight")
        self.scale = float(spec.params.get("scale", 1.0))
        self.norm = None if spec.params.get("norm") is None else self.prefix + str(spec.params["norm"])
        self.norm_eps = float(spec.params.get("norm_eps", 0.0))
        self.table = self.norm_w = None

    def tensors(self):
        out = [TensorSpec(self.name, (self.vocab, self.hidden), MATRIX)]
        if self.norm is not None:
            out.append(TensorSpec(self.norm, (self.hidden,), VECTOR, NORM_WEIGHT))
        return out

    def bind(self, weights):
        self.table = weights[self.name]
        if self.norm is not None:
            self.norm_w = weights[self.norm].to(torch.float32).contiguous()

    def kernel_modules(self):
        return ("elementwise",)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        h = ops.embed_gather(token_ids, self.table, scale=self.scale)
        return h if self.norm_w is None else ops.rmsnorm(h, self.norm_w, self.norm_eps, torch.float32)


class EmbeddingReinjection(StreamStep):
    """Adds onto the stream, in place and 32-bit: the step's token embeddings again (``add_embedding``: the table's rows
    times ``scale``, as the embedding made them) and row ``row`` of a learned table of vectors [rows, hidden_size]
    (``vector``: its tensor name; None for no vector).  A looped run of layers opens each of its passes with this.
    params: vocab_size, hidden_size, name (the embedding table), scale, add_embedding, vector, rows, row."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.vocab, self.hidden = int(p["vocab_size"]), int(p["hidden_size"])
        self.name = self.prefix + p.get("name", "embed_tokens.weight")
        self.scale = float(p.get("scale", 1.0))
        self.add_embedding = bool(p.get("add_embedding", True))
        self.vector = None if p.get("vector") is None else self.prefix + str(p["vector"])
        self.rows, self.row = int(p.get("rows", 1)), int(p.get("row", 0))
        if self.vector is not None and not 0 <= self.row < self.rows:
            raise ValueError(f"stream step '{self.vector}': row {self.row} of {self.rows}")
        self.table = self.vec = None

    def tensors(self):
        out = [TensorSpec(self.name, (self.vocab, self.hidden), MATRIX)] if self.add_embedding else []
        if self.vector is not None:
            out.append(TensorSpec(self.vector, (self.rows, self.hidden), VECTOR))
        return out

    def bind(self, weights):
        if self.add_embedding:
            self.table = weights[self.name]
        if self.vector is not None:
            self.vec = weights[self.vector][self.row].to(torch.float32).contiguous()

    def kernel_modules(self):
        return ("elementwise",)

    def forward(self, h, ctx):
        if self.add_embedding or self.vec is not None:
            ops.embed_add(h, ctx.token_ids if self.add_embedding else None, self.table, self.scale, self.vec)


class OutputHead(Part):
    """params: vocab_size, hidden_size, tied (True, False, or None: tied iff the head's tensor is absent),
    name, tied_to (name of the embedding table), scale (logits are multiplied by it; default 1), softcap (c > 0: logits
    become c * tanh(logits / c) after the scale; default 0: none)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = spec.params.get("tied")
        self.name = self.prefix + spec.params.get("name", "lm_head.weight")
        self.tied_to = spec.params["tied_to"]
        self.scale = float(spec.params.get("scale", 1.0))
        self.softcap = float(spec.params.get("softcap", 0.0) or 0.0)
        self.weight = None

    def tensors(self):
        # tied: a stored copy may be there and is not used; undecided: the tensor's presence decides
        return [TensorSpec(self.name, (self.vocab, self.hidden), MATRIX,
                           optional=self.tied is None, ignored=self.tied is True)]

    def bind(self, weights):
        if self.tied is True or (self.tied is None and self.name not in weights):
            self.weight = weights[self.tied_to]
        else:
            self.weight = weights[self.name]

    def kernel_modules(self):
        return ("elementwise", *linear_modules(self.runtime.dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.scale_softcap(linear(x, self.weight), self.scale, self.softcap)


register_embedding("token", TokenEmbedding)
register_head("linear", OutputHead)
register_stream_step("reinject_embedding", EmbeddingReinjection)
