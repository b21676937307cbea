"""Pre-norm residual block: h += mixer(norm1(h)); h += feed_forward(norm2(h))
(the reference: core/runtime.cpp:1015-1081; for this arrangement the second norm reads the
same tensor that the second residual sum starts from, :1066-1067).  The sums are folded into
the norms (each norm takes (h, delta), writes h + delta back and norms it) or, for parts that say
``adds_to_residual``, into the epilogue of the part's last matrix product (delta is then None) - or that product
comes back as a ``SplitSum``, sums over pieces of k that the next norm adds (``settle`` adds them for a norm that
does not say ``adds_split_sums``)."""
from __future__ import annotations

from dataclasses import replace

from .base import Block, NormedSum, ScaledSum
from .linear import settle
from .registry import build_part, register_block


class PreNormBlock(Block):
    """params: mixer_norm, ffn_norm (tensor-name stems of the two norms), mixer_prefix, ffn_prefix."""

    def __init__(self, spec, runtime, layer=None, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        px = spec.prefix
        self.norm1 = build_part("norm", replace(layer.norm, prefix=px + p.get("mixer_norm", "input_layernorm") + "."), runtime)
        self.norm2 = build_part("norm", replace(layer.norm, prefix=px + p.get("ffn_norm", "post_attention_layernorm") + "."), runtime)
        self.mixer = build_part("mixer", replace(layer.mixer, prefix=px + p.get("mixer_prefix", "self_attn") + "."),
                                runtime, position=position)
        self.ffn = build_part("feed_forward", replace(layer.feed_forward, prefix=px + p.get("ffn_prefix", "mlp") + "."), runtime)

    def parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    def tensors(self):
        return [t for part in self.parts() for t in part.tensors()]

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def kernel_modules(self):
        return tuple(m for part in self.parts() for m in part.kernel_modules())

    def forward(self, h, delta, ctx, cache):
        x = self.norm1.forward(h, settle(h, delta, self.norm1), write_sum=True)
        if self.mixer.adds_to_residual:
            delta = self.mixer.forward(x, ctx, cache, residual=h)
        else:
            delta = self.mixer.forward(x, ctx, cache)
        x = self.norm2.forward(h, settle(h, delta, self.norm2), write_sum=True)
        if self.ffn.adds_to_residual:
            delta = self.ffn.forward(x, ctx, residual=h)
        else:
            delta = self.ffn.forward(x, ctx)
        return h, delta


class OutputNormBlock(Block):
    """h += norm1(mixer(h)); h += norm2(feed_forward(h)): the sublayers read the stream itself and the norms sit on
    their outputs.  The stream and both sums are 32-bit; the norm kernel that adds onto the stream also hands back the
    stream in the dtype of the next product's operands, and the block leaves it in ``ctx.shared`` for the block after it.
    A layer without a feed-forward (``feed_forward`` None) has the first half only.
    params: mixer_norm, ffn_norm (the norms' tensor names after the layer's prefix), mixer_prefix, ffn_prefix."""

    def __init__(self, spec, runtime, layer=None, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        px = spec.prefix

        def norm(name):
            return build_part("norm", replace(layer.norm, prefix=px, params={**dict(layer.norm.params), "name": name}), runtime)

        self.norm1 = norm(p.get("mixer_norm", "norm1"))
        self.mixer = build_part("mixer", replace(layer.mixer, prefix=px + p.get("mixer_prefix", "mix") + "."),
                                runtime, position=position)
        self.ffn = self.norm2 = None
        if layer.feed_forward is not None:
            self.norm2 = norm(p.get("ffn_norm", "norm2"))
            self.ffn = build_part("feed_forward", replace(layer.feed_forward, prefix=px + p.get("ffn_prefix", "mlp") + "."), runtime)

    def parts(self):
        return [part for part in (self.norm1, self.mixer, self.norm2, self.ffn) if part is not None]

    def tensors(self):
        return [t for part in self.parts() for t in part.tensors()]

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def kernel_modules(self):
        return ("elementwise", *(m for part in self.parts() for m in part.kernel_modules()))

    def forward(self, h, delta, ctx, cache):
        from ..kernels import ops
        dtype = self.runtime.dtype
        if delta is not None:                                   # a block of another arrangement came before
            if hasattr(delta, "add_onto"):
                delta.add_onto(h)
            else:
                ops.add_inplace(h, delta)
        have = ctx.shared.get("stream_as_operand")
        x = have[1] if have is not None and have[0] is h else ops.bias_act(h, None, "none", dtype)
        x = self.norm1.add_normed(h, self.mixer.forward(x, ctx, cache), cast_dtype=dtype)
        if self.ffn is not None:
            x = self.norm2.add_normed(h, self.ffn.forward(x, ctx), cast_dtype=dtype)
        ctx.shared["stream_as_operand"] = (h, x)
        return h, None


class SandwichNormBlock(Block):
    """h += post1(mixer(pre1(h))); h += post2(feed_forward(pre2(h))): a norm in front of each sublayer and another on
    its output.  The normed output is not added here: it is handed on as a ``NormedSum``, so that the norm in front of
    the next sublayer (of this block, of the next block, or the model's last norm) adds it and norms the sum in one pass
    over the row.  A layer without a feed-forward (``feed_forward`` None) has the first half only.
    params: mixer_norm, mixer_post_norm, ffn_norm, ffn_post_norm (the norms' tensor names after the layer's prefix),
    mixer_prefix, ffn_prefix."""

    def __init__(self, spec, runtime, layer=None, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        px = spec.prefix

        def norm(name):
            return build_part("norm", replace(layer.norm, prefix=px, params={**dict(layer.norm.params), "name": name}), runtime)

        self.norm1, self.norm1b = norm(p.get("mixer_norm", "norm1")), norm(p.get("mixer_post_norm", "norm1b"))
        self.mixer = build_part("mixer", replace(layer.mixer, prefix=px + p.get("mixer_prefix", "mix") + "."),
                                runtime, position=position)
        self.ffn = self.norm2 = self.norm2b = None
        if layer.feed_forward is not None:
            self.norm2, self.norm2b = norm(p.get("ffn_norm", "norm2")), norm(p.get("ffn_post_norm", "norm2b"))
            self.ffn = build_part("feed_forward", replace(layer.feed_forward, prefix=px + p.get("ffn_prefix", "mlp") + "."), runtime)

    def parts(self):
        return [part for part in (self.norm1, self.mixer, self.norm1b, self.norm2, self.ffn, self.norm2b) if part is not None]

    def tensors(self):
        return [t for part in self.parts() for t in part.tensors()]

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def kernel_modules(self):
        return tuple(m for part in self.parts() for m in part.kernel_modules())

    def forward(self, h, delta, ctx, cache):
        x = self.norm1.forward(h, settle(h, delta, self.norm1), write_sum=True)
        delta = NormedSum(self.mixer.forward(x, ctx, cache), self.norm1b)
        if self.ffn is not None:
            x = self.norm2.forward(h, settle(h, delta, self.norm2), write_sum=True)
            delta = NormedSum(self.ffn.forward(x, ctx), self.norm2b)
        return h, delta


class ParallelResidualBlock(Block):
    """x = norm(h); h += mult * (mixer(x) + feed_forward(x)): one norm, both sublayers read its output, and their sum,
    times a constant, goes onto the stream.  The sum onto the stream is not made here: it is handed on as a
    ``ScaledSum``, so that the next norm (of the next block, or the model's last) multiplies, adds and norms in one pass
    over the row.  A feed-forward that can add its last product onto something adds it onto the mixer's output.  A layer
    without a feed-forward (``feed_forward`` None) has the mixer only.
    params: norm (the norm's tensor name after the layer's prefix), mixer_prefix, ffn_prefix, residual_mult (default 1)."""

    def __init__(self, spec, runtime, layer=None, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        px = spec.prefix
        self.mult = float(p.get("residual_mult", 1.0))
        self.norm1 = build_part("norm", replace(layer.norm, prefix=px, params={**dict(layer.norm.params), "name": p.get("norm", "norm1")}),
                                runtime)
        self.mixer = build_part("mixer", replace(layer.mixer, prefix=px + p.get("mixer_prefix", "mix") + "."),
                                runtime, position=position)
        self.ffn = None
        if layer.feed_forward is not None:
            self.ffn = build_part("feed_forward", replace(layer.feed_forward, prefix=px + p.get("ffn_prefix", "mlp") + "."), runtime)

    def parts(self):
        return [part for part in (self.norm1, self.mixer, self.ffn) if part is not None]

    def tensors(self):
        return [t for part in self.parts() for t in part.tensors()]

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def kernel_modules(self):
        return ("elementwise", *(m for part in self.parts() for m in part.kernel_modules()))

    def forward(self, h, delta, ctx, cache):
        x = self.norm1.forward(h, settle(h, delta, self.norm1), write_sum=True)
        y = self.mixer.forward(x, ctx, cache)
        if self.ffn is not None:
            if self.ffn.adds_to_residual:
                rest = self.ffn.forward(x, ctx, residual=y)     # None: added onto y in the last product's epilogue
                if rest is not None:
                    y = rest.add_onto(y) if hasattr(rest, "add_onto") else y.add_(rest)
            else:
                y = y.add_(self.ffn.forward(x, ctx))
        return h, ScaledSum(y, self.mult)


class PostNormBlock(Block):
    """h <- norm1(alpha * h + mixer(h)); h <- norm2(alpha * h + feed_forward(h)): the sublayers read the stream itself,
    and the stream is normed AFTER each sum, so that what a layer hands on is a normed row.  The stream, both sums and
    the norms are 32-bit; the norm kernel forms the sum, norms it, writes it back and also hands out the row in the
    dtype of the next product's operands.  A mixer that says ``reads_stream`` gets the 32-bit stream.  A layer without a
    feed-forward (``feed_forward`` None) has the first half only.
    params: mixer_norm, ffn_norm (the norms' tensor names after the layer's prefix), mixer_prefix, ffn_prefix, alpha
    (the constant on the stream in both sums; default 1)."""

    def __init__(self, spec, runtime, layer=None, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        px = spec.prefix
        self.alpha = float(p.get("alpha", 1.0))

        def norm(name):
            return build_part("norm", replace(layer.norm, prefix=px, params={**dict(layer.norm.params), "name": name}), runtime)

        self.norm1 = norm(p.get("mixer_norm", "norm1"))
        if not hasattr(self.norm1, "norm_sum"):
            raise ValueError(f"block '{px}': the norm '{layer.norm.kind}' cannot norm a sum in place")
        self.mixer = build_part("mixer", replace(layer.mixer, prefix=px + p.get("mixer_prefix", "mix") + "."),
                                runtime, position=position)
        self.ffn = self.norm2 = None
        if layer.feed_forward is not None:
            self.norm2 = norm(p.get("ffn_norm", "norm2"))
            self.ffn = build_part("feed_forward", replace(layer.feed_forward, prefix=px + p.get("ffn_prefix", "mlp") + "."), runtime)

    def parts(self):
        return [part for part in (self.norm1, self.mixer, self.norm2, self.ffn) if part is not None]

    def tensors(self):
        return [t for part in self.parts() for t in part.tensors()]

    def bind(self, weights):
        for part in self.parts():
            part.bind(weights)

    def kernel_modules(self):
        return ("elementwise", *(m for part in self.parts() for m in part.kernel_modules()))

    def forward(self, h, delta, ctx, cache):
        from ..kernels import ops
        dtype = self.runtime.dtype
        if delta is not None:                                   # a block of another arrangement came before
            if hasattr(delta, "add_onto"):
                delta.add_onto(h)
            else:
                ops.add_inplace(h, delta)
        if self.mixer.reads_stream:
            x = h
        else:
            have = ctx.shared.get("stream_as_operand")
            x = have[1] if have is not None and have[0] is h else ops.bias_act(h, None, "none", dtype)
        # the stream in the products' dtype is made where a feed-forward follows; the next block makes its own if it needs one
        x = self.norm1.norm_sum(h, self.mixer.forward(x, ctx, cache), self.alpha, cast_dtype=dtype if self.ffn is not None else None)
        ctx.shared.pop("stream_as_operand", None)
        if self.ffn is not None:
            self.norm2.norm_sum(h, self.ffn.forward(x, ctx), self.alpha)
        return h, None


register_block("pre_norm", PreNormBlock)
register_block("post_norm", PostNormBlock)
register_block("sandwich_norm", SandwichNormBlock)
register_block("output_norm", OutputNormBlock)
register_block("parallel_residual", ParallelResidualBlock)
