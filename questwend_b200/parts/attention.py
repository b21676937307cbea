"""Grouped-query attention over the paged cache, with optional per-head q/k norm, a position
encoding applied to q and k, and an optional window.  The reference's order (core/runtime.cpp:
1039-1058, 681-734): project, split heads, norm q and k (same eps), rotate, store k and v, attend
with scale 1/sqrt(head size), project back."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..kernels.limits import (conv_taps_refusal, head_dim_refusal, maps_attention_refusal, pool_attention_refusal,
                              shaped_attention_refusal)
from ..weights.manifest import MATRIX, NORM_WEIGHT, VECTOR, TensorSpec
from .base import KVSpec, Mixer, StateSpec, take_weight
from .linear import kernel_modules as linear_modules, linear, linear_onto
from .registry import register_mixer

FUSED_DECODE_MAX_BATCH = 16     # up to here a kernel less per layer pays (3-4 % of a small model's step); with more sequences
                                # every attention block repeating the work on q costs more than it saves (measured at 64).
                                # (Beyond a few rows a step's products change kernels too, so a step's arithmetic differs in
                                # its last bits between small and large batches anyway.)
DECODE_SPLIT_TOKENS = 256     # keys per run of the plain decode kernel; fixed, so results do not depend on the batch
                              # (the tensor-core kernel cuts by each sequence's own length: ops.attn_decode)


class GroupedQueryAttention(Mixer):
    """params: hidden_size, n_heads, n_kv_heads, head_dim, qk_norm (bool), norm_eps, window (0: none),
    scale (default 1/sqrt(head_dim)), names (optional overrides of the tensor names)."""

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv_heads = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("norm_eps", 0.0))
        self.window = int(p.get("window", 0) or 0)
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        self.position = position
        self.rotary_dim = getattr(position, "rotary_dim", 0) if position is not None else 0
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads are not a multiple of {self.n_kv_heads} key/value heads")
        refusal = head_dim_refusal(self.head_dim)           # now, and not at the first step with the weights loaded
        if refusal:
            raise ValueError(f"grouped-query attention '{self.prefix}': parameter 'head_dim': {refusal}")
        if self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} exceeds the head size {self.head_dim}")
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    def tensors(self):
        q, kv, hd, D = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, self.head_dim, self.hidden
        n = self.names
        out = [TensorSpec(self.prefix + n["q"], (q, D), MATRIX), TensorSpec(self.prefix + n["k"], (kv, D), MATRIX),
               TensorSpec(self.prefix + n["v"], (kv, D), MATRIX), TensorSpec(self.prefix + n["o"], (D, q), MATRIX)]
        if self.qk_norm:
            out += [TensorSpec(self.prefix + n["q_norm"], (hd,), VECTOR, NORM_WEIGHT),
                    TensorSpec(self.prefix + n["k_norm"], (hd,), VECTOR, NORM_WEIGHT)]
        return out

    def bind(self, weights):
        n, px = self.names, self.prefix
        # one fused projection: rows of q, then k, then v (a row concat, no change to the math).  The three sources are
        # taken out of ``weights`` (see ``take_weight``), so that a large model does not hold them twice until every layer
        # is bound.
        self.w_qkv = torch.cat([take_weight(weights, px + n[x]) for x in "qkv"], dim=0).contiguous()
        self.w_o = weights[px + n["o"]]
        if self.qk_norm:
            self.q_norm_w = weights[px + n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm_w = weights[px + n["k_norm"]].to(torch.float32).contiguous()

    def kernel_modules(self):
        mods = ["rope_kv", *linear_modules(self.runtime.dtype)]
        if ops.mma_attention_fits(self.runtime.dtype, self.head_dim, ops.PAGE_SIZE):
            mods.append("attention_mma")
            if ops.tc_attention_fits(self.runtime.dtype, self.head_dim, ops.PAGE_SIZE, self.n_heads // self.n_kv_heads):
                mods.append("attention_tc")
        else:
            mods.append("attention")
        return tuple(mods)

    def kv_spec(self):
        return KVSpec(self.n_kv_heads, self.head_dim, self.window)

    adds_to_residual = True

    def forward(self, x, ctx, cache, residual=None):
        qkv = linear(x, self.w_qkv)
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.prepare(ctx)
        table = ctx.page_tables[cache.group_id]
        if (ctx.single_token and ctx.n_seqs <= FUSED_DECODE_MAX_BATCH and self.rotary_dim in (0, self.head_dim)
                and ops.mma_attention_fits(cache.k_pool.dtype, self.head_dim, cache.k_pool.shape[2])):
            # one token for each of a few sequences on the tensor-core path: norm, rotation and cache write happen inside
            # the attention kernel
            att = ops.attn_decode_fused(qkv, self.q_norm_w, self.k_norm_w, cos, sin, self.eps, cache.k_pool, cache.v_pool,
                                        table, ctx.seq_len, self.scale, ctx.max_len, self.n_heads, self.n_kv_heads,
                                        self.head_dim, window=self.window, store_kv=cache.writable)
        else:
            q = ops.qk_norm_rope_store(qkv, self.q_norm_w, self.k_norm_w, cos, sin, ctx.tok_seq, ctx.tok_pos, table,
                                       cache.k_pool, cache.v_pool, self.n_heads, self.n_kv_heads, self.head_dim,
                                       self.rotary_dim, self.eps, store_kv=cache.writable)
            if ctx.single_token:
                att = ops.attn_decode(q, cache.k_pool, cache.v_pool, table, ctx.seq_len, self.scale, ctx.max_len,
                                      window=self.window, split_tokens=DECODE_SPLIT_TOKENS)
            else:
                att = ops.attn_prefill(q, cache.k_pool, cache.v_pool, table, ctx.cu_seqlens, ctx.pos0, ctx.max_new,
                                       self.scale, window=self.window)
        if residual is not None:
            return linear_onto(att, self.w_o, residual)     # None: the residual sum was made in the product's epilogue
        return linear(att, self.w_o)


class WindowPoolAttention(Mixer):
    """Grouped-query attention over a sliding window plus pooled blocks of what lies before it.  The query at position p
    sees the keys j with p - ``window`` < j <= p and, beside them, one key and value for each block of ``pool`` positions
    that lies wholly before the window (block b = positions b*pool .. b*pool + pool - 1, seen when b*pool + pool - 1 <=
    p - window): the means of the block's cached keys and values.  Tokens and blocks share one softmax.  Keys and values
    may differ in size.  Per-head RMS norm of q and k (``qk_norm``; one weight for all heads), a rotation of the first
    part of q and k, and (``rotate_values``) a rotation of every whole value by its own position before it is cached,
    undone on each head's output by the query's position.

    params: hidden_size, n_heads, n_kv_heads, head_dim, value_dim, qk_norm (bool), norm_eps, window (0: all keys, no
    blocks), pool (0: no blocks), scale (default 1/sqrt(head_dim)), rotate_values (bool), layout ("halves": pairs
    (i, i + n/2); "interleaved": (2i, 2i + 1)), names (optional overrides).  ``position``: the encoding of q and k, or a
    pair (q/k encoding, values' encoding); an encoding gives cos and sin [T, n/2].
    The cache: keys and values per token, and (with blocks) a second pair of pools with a row per complete block."""

    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}
    LAYOUTS = ("halves", "interleaved")

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.n_kv_heads = int(p["n_heads"]), int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim", self.head_dim))
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("norm_eps", 0.0))
        self.window = int(p.get("window", 0) or 0)
        self.pool = int(p.get("pool", 0) or 0) if self.window else 0
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.rotate_values = bool(p.get("rotate_values", False))
        self.layout = str(p.get("layout", "halves"))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        positions = position if isinstance(position, (tuple, list)) else (position, None)
        self.position, self.value_position = positions[0], (positions[1] if len(positions) > 1 else None)
        self.rotary_dim = getattr(self.position, "rotary_dim", 0) if self.position is not None else 0
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads are not a multiple of {self.n_kv_heads} key/value heads")
        if self.layout not in self.LAYOUTS:
            raise ValueError(f"attention '{self.prefix}': layout '{self.layout}' is not one of {', '.join(self.LAYOUTS)}")
        refusal = pool_attention_refusal(self.head_dim, self.value_dim)
        if refusal:
            raise ValueError(f"attention '{self.prefix}': {refusal}")
        if self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} exceeds the head size {self.head_dim}")
        if self.rotate_values and (self.value_position is None or getattr(self.value_position, "rotary_dim", 0) != self.value_dim):
            raise ValueError(f"attention '{self.prefix}': turned values need an encoding over all {self.value_dim} of a value")

    def tensors(self):
        q, kv, vv, D = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, self.n_kv_heads * self.value_dim, self.hidden
        n, px = self.names, self.prefix
        out = [TensorSpec(px + n["q"], (q, D), MATRIX), TensorSpec(px + n["k"], (kv, D), MATRIX),
               TensorSpec(px + n["v"], (vv, D), MATRIX), TensorSpec(px + n["o"], (D, self.n_heads * self.value_dim), MATRIX)]
        if self.qk_norm:
            out += [TensorSpec(px + n["q_norm"], (self.head_dim,), VECTOR, NORM_WEIGHT),
                    TensorSpec(px + n["k_norm"], (self.head_dim,), VECTOR, NORM_WEIGHT)]
        return out

    def bind(self, weights):
        n, px = self.names, self.prefix
        self.w_qkv = torch.cat([take_weight(weights, px + n[x]) for x in "qkv"], dim=0).contiguous()
        self.w_o = weights[px + n["o"]]
        self.q_norm_w = self.k_norm_w = None
        if self.qk_norm:
            self.q_norm_w = weights[px + n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm_w = weights[px + n["k_norm"]].to(torch.float32).contiguous()

    def kernel_modules(self):
        return ("attention_pool", "rope_kv", *linear_modules(self.runtime.dtype))

    def kv_spec(self):
        tokens = KVSpec(self.n_kv_heads, self.head_dim, self.window, value_dim=self.value_dim)
        if not self.pool:
            return tokens
        return (tokens, KVSpec(self.n_kv_heads, self.head_dim, self.window, value_dim=self.value_dim, stride=self.pool))

    def forward(self, x, ctx, cache):
        qkv = linear(x, self.w_qkv)
        cos = sin = cos_v = sin_v = None
        if self.position is not None and self.rotary_dim:
            cos, sin = self.position.prepare(ctx)
        if self.rotate_values:
            cos_v, sin_v = self.value_position.prepare(ctx)
        interleaved = self.layout == "interleaved"
        table = ctx.page_tables[cache.group_id]
        q = ops.pool_prep(qkv, self.q_norm_w, self.k_norm_w, cos, sin, cos_v, sin_v, ctx, table, cache.k_pool, cache.v_pool,
                          self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim, self.rotary_dim, interleaved, self.eps,
                          store_kv=cache.writable)
        pk = pv = block_table = None
        if self.pool:
            blocks = cache.more[0]
            pk, pv, block_table = blocks.k_pool, blocks.v_pool, ctx.page_tables[blocks.group_id]
            if cache.writable:
                ops.pool_update(cache.k_pool, cache.v_pool, pk, pv, table, block_table, ctx, self.pool)
        att = ops.pool_attention(q, cache.k_pool, cache.v_pool, pk, pv, table, block_table, ctx, cos_v, sin_v, self.scale,
                                 self.window, self.pool, interleaved)
        return linear(att, self.w_o)


class ScoreMapsAttention(Mixer):
    """Grouped-query softmax attention whose heads carry ``maps`` score maps (1 or 2) over the same values.  A query head
    has ``maps`` query vectors of ``head_dim`` values laid out one after the other, a key head as many key vectors; each
    map is an attention of its own (score = q . k * ``scale``, then ``softcap`` * tanh(score / ``softcap``) if that is
    > 0, a causal mask, and with ``chunk`` > 0 only the keys of the query's own block of ``chunk`` positions, counted
    from the sequence's start).  With two maps the head's output is differential: a1 - lambda * a2 with
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``diff`` (four learned vectors of the layer), divided by its root mean
    square over the value size (eps inside the root) and multiplied by 1 - ``diff``.  In front of the scores, in this
    order and each optional: biases on q, k and v, a short causal convolution over time on every channel of q, k and v
    (``conv`` taps, no activation; its last inputs are per-sequence state), an RMS norm of every map of q and k with a
    weight shared by heads and maps, and a rotation of the first part of every map.

    params: hidden_size, n_heads, n_kv_heads, head_dim, value_dim, maps (default 1), biases (q, k, v), out_bias, conv
    (0: none), qk_norm, norm_eps, scale (default 1/sqrt(head_dim)), softcap (0: none), chunk (0: plain causal), diff,
    layout ("halves": pairs (i, i + n/2); "interleaved": (2i, 2i + 1)), names (optional overrides).  ``position``: an
    encoding that gives cos and sin [T, n/2].
    The cache: keys (all maps of a head in one row) and values per token; with a convolution also its tail."""

    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
             "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "q_norm": "q.norm", "k_norm": "k.norm",
             "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
    LAYOUTS = ("halves", "interleaved")

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.n_kv_heads = int(p["n_heads"]), int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim", self.head_dim))
        self.maps = int(p.get("maps", 1))
        self.biases, self.out_bias = bool(p.get("biases", False)), bool(p.get("out_bias", False))
        self.taps = int(p.get("conv", 0) or 0)
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("norm_eps", 0.0))
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.chunk = int(p.get("chunk", 0) or 0)
        self.diff = float(p.get("diff", 0.0))
        self.layout = str(p.get("layout", "halves"))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        self.position = position[0] if isinstance(position, (tuple, list)) else position
        self.rotary_dim = getattr(self.position, "rotary_dim", 0) if self.position is not None else 0
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads are not a multiple of {self.n_kv_heads} key/value heads")
        if self.layout not in self.LAYOUTS:
            raise ValueError(f"attention '{self.prefix}': layout '{self.layout}' is not one of {', '.join(self.LAYOUTS)}")
        for refusal in (maps_attention_refusal(self.maps, self.head_dim, self.value_dim),
                        conv_taps_refusal(self.taps) if self.taps else None):
            if refusal:
                raise ValueError(f"attention '{self.prefix}': {refusal}")
        if self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} exceeds the map size {self.head_dim}")
        self.n_q = self.n_heads * self.maps * self.head_dim
        self.n_k = self.n_kv_heads * self.maps * self.head_dim
        self.n_v = self.n_kv_heads * self.value_dim
        self.channels = self.n_q + self.n_k + self.n_v
        self.lam = 0.0

    def tensors(self):
        n, px, D = self.names, self.prefix, self.hidden
        sizes = {"q": self.n_q, "k": self.n_k, "v": self.n_v}
        out = [TensorSpec(px + n[x], (sizes[x], D), MATRIX) for x in "qkv"]
        out.append(TensorSpec(px + n["o"], (D, self.n_heads * self.value_dim), MATRIX))
        if self.biases:
            out += [TensorSpec(px + n[x + "_bias"], (sizes[x],), VECTOR) for x in "qkv"]
        if self.out_bias:
            out.append(TensorSpec(px + n["o_bias"], (D,), VECTOR))
        if self.taps:
            out += [TensorSpec(px + n[x + "_conv"], (sizes[x], self.taps), VECTOR) for x in "qkv"]
        if self.qk_norm:
            out += [TensorSpec(px + n["q_norm"], (self.head_dim,), VECTOR, NORM_WEIGHT),
                    TensorSpec(px + n["k_norm"], (self.head_dim,), VECTOR, NORM_WEIGHT)]
        if self.maps == 2:
            out += [TensorSpec(px + n[x], (self.head_dim,), VECTOR) for x in ("lq1", "lk1", "lq2", "lk2")]
        return out

    def bind(self, weights):
        n, px = self.names, self.prefix

        def f32(name):
            return weights[px + n[name]].to(torch.float32).contiguous()

        self.w_qkv = torch.cat([take_weight(weights, px + n[x]) for x in "qkv"], dim=0).contiguous()
        self.w_o = weights[px + n["o"]]
        self.b_qkv = torch.cat([f32(x + "_bias") for x in "qkv"]).contiguous() if self.biases else None
        self.b_o = f32("o_bias") if self.out_bias else None
        self.conv_w = torch.cat([f32(x + "_conv") for x in "qkv"], dim=0).contiguous() if self.taps else None
        self.q_norm_w = f32("q_norm") if self.qk_norm else None
        self.k_norm_w = f32("k_norm") if self.qk_norm else None
        if self.maps == 2:      # one number for the layer, made once, in 64-bit on the host
            lq1, lk1, lq2, lk2 = (weights[px + n[x]].to(torch.float64).cpu() for x in ("lq1", "lk1", "lq2", "lk2"))
            self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff

    def kernel_modules(self):
        mods = ["attention_maps", "rope_kv", "elementwise", *(("recurrent",) if self.taps else ()), *linear_modules(self.runtime.dtype)]
        if (self.maps == 1 and self.softcap <= 0.0 and self.head_dim == self.value_dim
                and ops.tc_attention_fits(self.runtime.dtype, self.head_dim, ops.PAGE_SIZE, self.n_heads // self.n_kv_heads)):
            mods.append("attention_tc")         # prompts of one uncapped map with keys and values of 64 or 128
        return tuple(mods)

    def kv_spec(self):
        return KVSpec(self.n_kv_heads, self.maps * self.head_dim, 0, value_dim=self.value_dim)

    def state_spec(self):
        return StateSpec((self.taps - 1, self.channels), torch.float32) if self.taps > 1 else None

    def forward(self, x, ctx, cache):
        qkv = linear(x, self.w_qkv)
        bias = self.b_qkv
        if self.taps:
            tail = cache.state if self.taps > 1 else qkv.new_zeros((1, 0, self.channels))
            qkv = ops.short_conv(qkv, 0, self.channels, self.conv_w, None, tail, ctx, activation=False,
                                 update_tail=cache.writable, in_bias=bias)
            bias = None
        cos = sin = None
        if self.position is not None and self.rotary_dim:
            cos, sin = self.position.prepare(ctx)
        table = ctx.page_tables[cache.group_id]
        q = ops.maps_prep(qkv, bias, self.q_norm_w, self.k_norm_w, cos, sin, ctx, table, cache.k_pool, cache.v_pool,
                          self.n_heads, self.n_kv_heads, self.maps, self.head_dim, self.value_dim, self.rotary_dim,
                          self.layout == "interleaved", self.eps, store_kv=cache.writable)
        two = self.maps == 2
        att = ops.maps_attention(q, cache.k_pool, cache.v_pool, table, ctx, self.maps, self.scale, softcap=self.softcap,
                                 chunk=self.chunk, lam=self.lam, norm_out=two, eps=self.eps,
                                 out_scale=(1.0 - self.diff) if two else 1.0)
        out = linear(att, self.w_o)
        return ops.bias_act(out, self.b_o, "none", torch.float32) if self.b_o is not None else out


class ShapedScoreAttention(Mixer):
    """Grouped-query softmax attention whose scores are shaped head by head, each step optional and a parameter.  In
    front of the scores: biases on q and k (and v), an RMS norm of every head of q and k with a weight shared by the
    heads, a rotation of the first part of every head.  ``values_from_keys``: there is no value projection; a token's
    value is the raw output of its key projection (with its bias), ahead of the key's norm and turn.  score = q . k * ``scale``, times a learned
    number per head (``head_temperature``), capped (``softcap``: c tanh(s / c)), minus slope_h * (i - j) with
    slope_h = 2^(-``slope_base`` (h + 1) / H) (``slope_base`` > 0); causal, and within the last ``window`` positions if
    that is > 0; ``sink``: a learned number per head whose exponential joins the softmax's denominator (no key, no value).
    ``head_mix``: a learned [H, H] matrix mixes the heads' weights after the softmax, w'_h = sum_g M[h, g] w_g, each head
    still reading its own value head.  ``head_gate``: head h's output times sigmoid(W_g h)_h, one number per head.

    params: hidden_size, n_heads, n_kv_heads, head_dim, value_dim, biases, values_from_keys, qk_norm, norm_eps, scale
    (default 1/sqrt(head_dim)), head_temperature, softcap (0: none), slope_base (0: none), window (0: all keys), sink,
    head_mix, head_gate, layout ("halves": pairs (i, i + n/2); "interleaved": (2i, 2i + 1)), names (optional overrides).
    ``position``: an encoding that gives cos and sin [T, n/2], or None.  The cache: keys and values per token."""

    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "q_norm": "q.norm",
             "k_norm": "k.norm", "temp": "temp", "sink": "sink", "mix": "talk", "gate": "g"}
    LAYOUTS = ("halves", "interleaved")

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads, self.n_kv_heads = int(p["n_heads"]), int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.value_dim = int(p.get("value_dim", self.head_dim))
        self.biases = bool(p.get("biases", False))
        self.values_from_keys = bool(p.get("values_from_keys", False))
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("norm_eps", 0.0))
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.head_temperature = bool(p.get("head_temperature", False))
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.slope_base = float(p.get("slope_base", 0.0) or 0.0)
        self.window = int(p.get("window", 0) or 0)
        self.sink, self.head_mix, self.head_gate = (bool(p.get(k, False)) for k in ("sink", "head_mix", "head_gate"))
        self.layout = str(p.get("layout", "halves"))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        self.position = position[0] if isinstance(position, (tuple, list)) else position
        self.rotary_dim = getattr(self.position, "rotary_dim", 0) if self.position is not None else 0
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads are not a multiple of {self.n_kv_heads} key/value heads")
        if self.layout not in self.LAYOUTS:
            raise ValueError(f"attention '{self.prefix}': layout '{self.layout}' is not one of {', '.join(self.LAYOUTS)}")
        refusal = shaped_attention_refusal(self.head_dim, self.value_dim)
        if refusal:
            raise ValueError(f"attention '{self.prefix}': {refusal}")
        if self.values_from_keys and self.value_dim != self.head_dim:
            raise ValueError(f"attention '{self.prefix}': values that are the keys have the keys' size {self.head_dim}, "
                             f"not {self.value_dim}")
        if self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} exceeds the head size {self.head_dim}")
        self.n_q = self.n_heads * self.head_dim
        self.n_k = self.n_kv_heads * self.head_dim
        self.n_v = 0 if self.values_from_keys else self.n_kv_heads * self.value_dim
        self.temp = self.sinks = self.mix = self.slopes = None

    def _projections(self):
        return "qk" if self.values_from_keys else "qkv"

    def tensors(self):
        n, px, D, H = self.names, self.prefix, self.hidden, self.n_heads
        sizes = {"q": self.n_q, "k": self.n_k, "v": self.n_v}
        out = [TensorSpec(px + n[x], (sizes[x], D), MATRIX) for x in self._projections()]
        out.append(TensorSpec(px + n["o"], (D, H * self.value_dim), MATRIX))
        if self.biases:
            out += [TensorSpec(px + n[x + "_bias"], (sizes[x],), VECTOR) for x in self._projections()]
        if self.qk_norm:
            out += [TensorSpec(px + n["q_norm"], (self.head_dim,), VECTOR, NORM_WEIGHT),
                    TensorSpec(px + n["k_norm"], (self.head_dim,), VECTOR, NORM_WEIGHT)]
        if self.head_temperature:
            out.append(TensorSpec(px + n["temp"], (H,), VECTOR, NORM_WEIGHT))
        if self.sink:
            out.append(TensorSpec(px + n["sink"], (H,), VECTOR))
        if self.head_mix:
            out.append(TensorSpec(px + n["mix"], (H, H), VECTOR))
        if self.head_gate:
            out.append(TensorSpec(px + n["gate"], (H, D), MATRIX))
        return out

    def bind(self, weights):
        n, px, H = self.names, self.prefix, self.n_heads

        def f32(name):
            return weights[px + n[name]].to(torch.float32).contiguous()

        # one projection for everything that reads the mixer's input: q | k | (v) | (gate)
        mats = [take_weight(weights, px + n[x]) for x in self._projections()]
        if self.head_gate:
            mats.append(take_weight(weights, px + n["gate"]))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = weights[px + n["o"]]
        self.b_in = torch.cat([f32(x + "_bias") for x in self._projections()]).contiguous() if self.biases else None
        self.q_norm_w = f32("q_norm") if self.qk_norm else None
        self.k_norm_w = f32("k_norm") if self.qk_norm else None
        self.temp = f32("temp") if self.head_temperature else None
        self.sinks = f32("sink") if self.sink else None
        self.mix = f32("mix") if self.head_mix else None
        if self.slope_base > 0:
            slopes = [2.0 ** (-self.slope_base * (h + 1) / H) for h in range(H)]
            self.slopes = torch.tensor(slopes, dtype=torch.float32, device=self.w_o.device)

    def kernel_modules(self):
        mods = ["attention_bias", "rope_kv", *linear_modules(self.runtime.dtype)]
        if (not (self.head_temperature or self.softcap > 0.0 or self.head_mix or self.head_gate) and self.head_dim == self.value_dim
                and ops.tc_attention_fits(self.runtime.dtype, self.head_dim, ops.PAGE_SIZE, self.n_heads // self.n_kv_heads)):
            mods.append("attention_tc")         # prompts whose scores a distance bias, a window and a sink shape, keys and values of 64 or 128
        return tuple(mods)

    def kv_spec(self):
        return KVSpec(self.n_kv_heads, self.head_dim, self.window, value_dim=self.value_dim)

    def forward(self, x, ctx, cache):
        proj = linear(x, self.w_in)
        cos = sin = None
        if self.position is not None and self.rotary_dim:
            cos, sin = self.position.prepare(ctx)
        table = ctx.page_tables[cache.group_id]
        q = ops.bias_prep(proj, self.b_in, self.q_norm_w, self.k_norm_w, cos, sin, ctx, table, cache.k_pool, cache.v_pool,
                          self.n_heads, self.n_kv_heads, self.head_dim, self.value_dim, self.rotary_dim,
                          self.layout == "interleaved", self.eps, store_kv=cache.writable,
                          values_are_keys=self.values_from_keys)
        att = ops.bias_attention(q, cache.k_pool, cache.v_pool, table, ctx, self.scale, head_scale=self.temp,
                                 softcap=self.softcap, slopes=self.slopes, window=self.window, sinks=self.sinks,
                                 head_mix=self.mix, gate=proj if self.head_gate else None,
                                 gate_col0=self.n_q + self.n_k + self.n_v)
        return linear(att, self.w_o)


register_mixer("gqa", GroupedQueryAttention)
register_mixer("shaped_score_attention", ShapedScoreAttention)
register_mixer("window_pool_attention", WindowPoolAttention)
register_mixer("score_maps_attention", ScoreMapsAttention)
