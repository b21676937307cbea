"""Mixers that carry a state of fixed size from token to token instead of keys and values: the state-space
recurrence of Mamba-2, the gated delta rule with a decay per key channel or per head, gated linear attention (a decay per
key channel, a plain outer-product write), retention (the same write with a fixed decay per head and rotated queries and
keys), and the recurrent block around a real-gated linear recurrent unit (one number of state per channel).  All keep, per sequence, a 32-bit
state matrix per head and the last inputs of a short causal convolution, in the cache's per-slot state rows; a
prompt and a single token run through the same kernels (``csrc/recurrent.cu``).  The projections are matrix
products in the engine's dtype with 32-bit results; everything between them is 32-bit.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.limits import conv_taps_refusal, state_matrix_refusal
from ..weights.manifest import MATRIX, NORM_WEIGHT, VECTOR, TensorSpec
from .base import Mixer, StateSpec, take_weight
from .linear import kernel_modules as linear_modules, linear
from .registry import register_mixer


def _f32(weights, name):
    return weights[name].to(torch.float32).contiguous()


class Mamba2Mixer(Mixer):
    """Mamba-2.  One projection gives z | x | B | C | dt; x, B and C pass a causal convolution (with bias) and SiLU;
    per head h (group h // (heads / groups)):  dt = softplus(dt + dt_bias_h);  S = exp(-exp(A_log_h) dt) S + dt B x^T;
    y = S^T C + D_h x;  then y * silu(z), an RMS norm over ``norm_groups`` equal parts of the row, times the norm's
    weight, and the output projection.

    params: hidden_size, heads, vdim, state, groups, norm_groups, conv (taps), norm_eps, names (optional overrides).
    State per sequence: the convolution's last taps - 1 inputs [taps - 1, channels] and S, stored [heads, vdim, state]."""

    NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
             "norm": "norm", "out": "o"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.vdim, self.n_state = int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.groups, self.norm_groups, self.taps = int(p["groups"]), int(p["norm_groups"]), int(p["conv"])
        self.eps = float(p["norm_eps"])
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.n_state
        if self.heads % self.groups:
            raise ValueError(f"mamba2 '{self.prefix}': {self.heads} heads are not a multiple of {self.groups} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"mamba2 '{self.prefix}': {self.inner} values cannot be normed in {self.norm_groups} equal parts")
        for refusal in (conv_taps_refusal(self.taps), state_matrix_refusal(self.n_state, self.vdim)):
            if refusal:
                raise ValueError(f"mamba2 '{self.prefix}': {refusal}")

    def tensors(self):
        n, px, H = self.names, self.prefix, self.heads
        return [TensorSpec(px + n["in"], (2 * self.inner + 2 * self.groups * self.n_state + H, self.hidden), MATRIX),
                TensorSpec(px + n["conv"], (self.channels, self.taps), VECTOR),
                TensorSpec(px + n["conv_bias"], (self.channels,), VECTOR),
                TensorSpec(px + n["dt_bias"], (H,), VECTOR), TensorSpec(px + n["A_log"], (H,), VECTOR),
                TensorSpec(px + n["D"], (H,), VECTOR, NORM_WEIGHT),
                TensorSpec(px + n["norm"], (self.inner,), VECTOR, NORM_WEIGHT),
                TensorSpec(px + n["out"], (self.hidden, self.inner), MATRIX)]

    def bind(self, weights):
        n, px = self.names, self.prefix
        self.w_in, self.w_out = weights[px + n["in"]], weights[px + n["out"]]
        self.conv_w, self.conv_b = _f32(weights, px + n["conv"]), _f32(weights, px + n["conv_bias"])
        self.dt_bias, self.a_log, self.d_skip = (_f32(weights, px + n[k]) for k in ("dt_bias", "A_log", "D"))
        self.norm_w = _f32(weights, px + n["norm"])

    def kernel_modules(self):
        return ("recurrent", *linear_modules(self.runtime.dtype))

    def state_spec(self):
        return (StateSpec((self.taps - 1, self.channels), torch.float32),
                StateSpec((self.heads, self.vdim, self.n_state), torch.float32))       # column by column

    def forward(self, x, ctx, cache):
        tail, state = cache.state
        proj = linear(x, self.w_in)                                   # z | x B C | dt, 32-bit
        xbc = ops.short_conv(proj, self.inner, self.channels, self.conv_w, self.conv_b, tail, ctx,
                             update_tail=cache.writable)
        y = ops.ssm_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.d_skip, state, ctx,
                         self.heads, self.vdim, self.n_state, self.groups, write_state=cache.writable)
        g = ops.gated_part_norm(y, proj, 0, self.norm_w, self.norm_groups, self.eps, gate_first=True,
                                out_dtype=self.runtime.dtype)
        return linear(g, self.w_out)


class GatedDeltaMixer(Mixer):
    """The gated delta rule with one decay per head and key channel.  q and k (``key_heads`` heads of ``key_dim``) and v
    (``heads`` heads of ``vdim``) each pass a causal convolution (no bias) and SiLU; q and k become unit vectors per head
    (x / sqrt(sum x^2 + ``unit_eps``)), q times key_dim^-1/2; beta = sigmoid(W_b h); decay = exp(-exp(A_log_h) *
    softplus(W_a2 W_a1 h + dt_bias)) per (head, key channel).  Per head (its q/k head is h // (heads / key_heads)):
    S = decay[:, None] S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q.  Each head's o is RMS-normed over vdim,
    times a weight shared by the heads, times sigmoid(W_g2 W_g1 h); then the output projection.

    params: hidden_size, heads, key_heads, key_dim, vdim, conv (taps), decay_rank, gate_rank, norm_eps, unit_eps
    (default 1e-6), names.  State per sequence: the convolutions' last taps - 1 inputs and S, stored [heads, vdim, key_dim]."""

    NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b",
             "A_log": "A_log", "decay_down": "a1", "decay_up": "a2", "dt_bias": "dt_bias", "gate_down": "g1",
             "gate_up": "g2", "norm": "norm", "out": "o"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.key_heads = int(p["heads"]), int(p["key_heads"])
        self.key_dim, self.vdim, self.taps = int(p["key_dim"]), int(p["vdim"]), int(p["conv"])
        self.decay_rank, self.gate_rank = int(p["decay_rank"]), int(p["gate_rank"])
        self.eps, self.unit_eps = float(p["norm_eps"]), float(p.get("unit_eps", 1e-6))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        if self.heads % self.key_heads:
            raise ValueError(f"gated delta rule '{self.prefix}': {self.heads} heads are not a multiple of "
                             f"{self.key_heads} query/key heads")
        for refusal in (conv_taps_refusal(self.taps), state_matrix_refusal(self.key_dim, self.vdim)):
            if refusal:
                raise ValueError(f"gated delta rule '{self.prefix}': {refusal}")
        self.n_qk = self.key_heads * self.key_dim
        self.channels = 2 * self.n_qk + self.heads * self.vdim

    def tensors(self):
        n, px, D, H = self.names, self.prefix, self.hidden, self.heads
        return [TensorSpec(px + n["q"], (self.n_qk, D), MATRIX), TensorSpec(px + n["q_conv"], (self.n_qk, self.taps), VECTOR),
                TensorSpec(px + n["k"], (self.n_qk, D), MATRIX), TensorSpec(px + n["k_conv"], (self.n_qk, self.taps), VECTOR),
                TensorSpec(px + n["v"], (H * self.vdim, D), MATRIX),
                TensorSpec(px + n["v_conv"], (H * self.vdim, self.taps), VECTOR),
                TensorSpec(px + n["beta"], (H, D), MATRIX), TensorSpec(px + n["A_log"], (H,), VECTOR),
                TensorSpec(px + n["norm"], (self.vdim,), VECTOR, NORM_WEIGHT),
                TensorSpec(px + n["decay_down"], (self.decay_rank, D), MATRIX),
                TensorSpec(px + n["decay_up"], (H * self.key_dim, self.decay_rank), MATRIX),
                TensorSpec(px + n["dt_bias"], (H * self.key_dim,), VECTOR),
                TensorSpec(px + n["gate_down"], (self.gate_rank, D), MATRIX),
                TensorSpec(px + n["gate_up"], (H * self.vdim, self.gate_rank), MATRIX),
                TensorSpec(px + n["out"], (D, H * self.vdim), MATRIX)]

    def bind(self, weights):
        n, px = self.names, self.prefix
        # one projection for everything that reads the stream: q | k | v | beta | decay latent | gate latent
        self.w_in = torch.cat([take_weight(weights, px + n[k]) for k in ("q", "k", "v", "beta", "decay_down", "gate_down")],
                              dim=0).contiguous()
        self.conv_w = torch.cat([_f32(weights, px + n[k]) for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.w_decay_up, self.w_gate_up, self.w_out = (weights[px + n[k]] for k in ("decay_up", "gate_up", "out"))
        self.a_log, self.dt_bias, self.norm_w = (_f32(weights, px + n[k]) for k in ("A_log", "dt_bias", "norm"))

    def kernel_modules(self):
        return ("recurrent", "elementwise", *linear_modules(self.runtime.dtype))

    def state_spec(self):
        return (StateSpec((self.taps - 1, self.channels), torch.float32),
                StateSpec((self.heads, self.vdim, self.key_dim), torch.float32))       # column by column

    def forward(self, x, ctx, cache):
        tail, state = cache.state
        dtype, C, H = self.runtime.dtype, self.channels, self.heads
        proj = linear(x, self.w_in)
        qkv = ops.short_conv(proj, 0, C, self.conv_w, None, tail, ctx, update_tail=cache.writable)
        a_raw = linear(ops.bias_act(proj, None, "none", dtype, C + H, self.decay_rank), self.w_decay_up)
        o = ops.delta_rule(qkv, proj, C, a_raw, self.dt_bias, self.a_log, state, ctx, H, self.key_heads, self.key_dim,
                           self.vdim, self.unit_eps, self.key_dim ** -0.5, write_state=cache.writable)
        gate = linear(ops.bias_act(proj, None, "none", dtype, C + H + self.decay_rank, self.gate_rank), self.w_gate_up)
        g = ops.gated_part_norm(o, gate, 0, self.norm_w, H, self.eps, gate_first=False, out_dtype=dtype)
        return linear(g, self.w_out)


class RGLRUMixer(Mixer):
    """A recurrent block around a real-gated linear recurrent unit.  Two branches of ``width`` channels read the
    mixer's input h: y = gelu_tanh(W_y h + b_y), and u = conv(W_x h + b_x), a causal convolution per channel with a
    bias and no activation (zeros before a sequence's start).  The channels of u are cut into ``blocks`` equal parts;
    per part b two gates r = sigmoid(A_b u_b + a_b) and i = sigmoid(I_b u_b + i_b) with square matrices.  Per channel
    log a = -``sharpness`` * r * softplus(lam), S = a S + sqrt(1 - a^2) * i * u from S = 0, the first token like every
    other; the output is W_o (S * y).  Gates, decays and the state are 32-bit.

    params: hidden_size, width, blocks, conv (taps), sharpness (default 8), names (optional overrides).
    State per sequence: the convolution's last taps - 1 inputs [taps - 1, width] and S [width]."""

    NAMES = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b",
             "decay_gate": "ra", "decay_gate_bias": "ra.b", "input_gate": "ri", "input_gate_bias": "ri.b", "lam": "lam",
             "out": "o"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden, self.width = int(p["hidden_size"]), int(p["width"])
        self.blocks, self.taps = int(p["blocks"]), int(p["conv"])
        self.sharpness = float(p.get("sharpness", 8.0))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        if self.blocks <= 0 or self.width % self.blocks:
            raise ValueError(f"rglru '{self.prefix}': {self.width} channels cannot be cut into {self.blocks} equal blocks")
        refusal = conv_taps_refusal(self.taps)
        if refusal:
            raise ValueError(f"rglru '{self.prefix}': {refusal}")

    def tensors(self):
        n, px, W, D, nb = self.names, self.prefix, self.width, self.hidden, self.blocks
        bw = W // nb
        return [TensorSpec(px + n["y"], (W, D), MATRIX), TensorSpec(px + n["y_bias"], (W,), VECTOR),
                TensorSpec(px + n["x"], (W, D), MATRIX), TensorSpec(px + n["x_bias"], (W,), VECTOR),
                TensorSpec(px + n["conv"], (W, self.taps), VECTOR), TensorSpec(px + n["conv_bias"], (W,), VECTOR),
                TensorSpec(px + n["decay_gate"], (nb, bw, bw), MATRIX), TensorSpec(px + n["decay_gate_bias"], (nb, bw), VECTOR),
                TensorSpec(px + n["input_gate"], (nb, bw, bw), MATRIX), TensorSpec(px + n["input_gate_bias"], (nb, bw), VECTOR),
                TensorSpec(px + n["lam"], (W,), VECTOR), TensorSpec(px + n["out"], (D, W), MATRIX)]

    def bind(self, weights):
        n, px = self.names, self.prefix
        # one projection for both branches: y | x
        self.w_in = torch.cat([take_weight(weights, px + n["y"]), take_weight(weights, px + n["x"])], dim=0).contiguous()
        self.w_out = weights[px + n["out"]]
        self.b_y, self.b_x, self.conv_w, self.conv_b, self.lam = (
            _f32(weights, px + n[k]) for k in ("y_bias", "x_bias", "conv", "conv_bias", "lam"))
        self.w_decay_gate, self.w_input_gate = (weights[px + n[k]].contiguous() for k in ("decay_gate", "input_gate"))
        self.b_decay_gate, self.b_input_gate = (_f32(weights, px + n[k]) for k in ("decay_gate_bias", "input_gate_bias"))

    def kernel_modules(self):
        return ("recurrent", "rglru", *linear_modules(self.runtime.dtype))

    def state_spec(self):
        return (StateSpec((self.taps - 1, self.width), torch.float32), StateSpec((self.width,), torch.float32))

    def forward(self, x, ctx, cache):
        tail, state = cache.state
        W = self.width
        proj = linear(x, self.w_in)                                   # y | x before their biases, 32-bit
        u = ops.short_conv(proj, W, W, self.conv_w, self.conv_b, tail, ctx, activation=False, update_tail=cache.writable,
                           in_bias=self.b_x)
        r, i = ops.block_gates(u, self.w_decay_gate, self.b_decay_gate, self.w_input_gate, self.b_input_gate)
        g = ops.rglru_scan(u, r, i, self.lam, proj, 0, self.b_y, state, ctx, self.sharpness, self.runtime.dtype,
                           write_state=cache.writable)
        return linear(g, self.w_out)


class GatedLinearAttentionMixer(Mixer):
    """Linear attention with a decay per head and key channel.  q = W_q h * ``q_scale`` and k = W_k h (heads x key_dim),
    v = W_v h (heads x vdim); the decay is alpha = sigmoid(z)^(1 / ``tau``) with z = W_a2 (W_a1 h) + b (a low-rank
    projection, heads x key_dim).  Per head S <- diag(alpha) S + k v^T from S = 0 and o = S^T q; each head's o is
    RMS-normed over vdim with one weight shared by the heads, multiplied by silu(W_g h), and projected by W_o.  The
    state, the decays (formed as exp(log_sigmoid(z) / tau)) and the norm are 32-bit.

    params: hidden_size, heads, key_dim, vdim, decay_rank, tau, norm_eps, q_scale (default key_dim^-1/2), names (optional
    overrides).  State per sequence: S, stored [heads, vdim, key_dim]."""

    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "decay_down": "a1", "decay_up": "a2", "decay_bias": "a2.b",
             "norm": "norm", "out": "o"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.key_dim, self.vdim = int(p["heads"]), int(p["key_dim"]), int(p["vdim"])
        self.decay_rank = int(p["decay_rank"])
        self.tau, self.eps = float(p["tau"]), float(p["norm_eps"])
        self.q_scale = float(p.get("q_scale", self.key_dim ** -0.5))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        refusal = state_matrix_refusal(self.key_dim, self.vdim)
        if refusal:
            raise ValueError(f"gated linear attention '{self.prefix}': {refusal}")
        if not self.tau > 0:
            raise ValueError(f"gated linear attention '{self.prefix}': tau must be positive, got {self.tau}")
        self.n_qk = self.heads * self.key_dim
        self.n_v = self.heads * self.vdim

    def tensors(self):
        n, px, D = self.names, self.prefix, self.hidden
        return [TensorSpec(px + n["q"], (self.n_qk, D), MATRIX), TensorSpec(px + n["k"], (self.n_qk, D), MATRIX),
                TensorSpec(px + n["v"], (self.n_v, D), MATRIX), TensorSpec(px + n["gate"], (self.n_v, D), MATRIX),
                TensorSpec(px + n["out"], (D, self.n_v), MATRIX),
                TensorSpec(px + n["norm"], (self.vdim,), VECTOR, NORM_WEIGHT),
                TensorSpec(px + n["decay_down"], (self.decay_rank, D), MATRIX),
                TensorSpec(px + n["decay_up"], (self.n_qk, self.decay_rank), MATRIX),
                TensorSpec(px + n["decay_bias"], (self.n_qk,), VECTOR)]

    def bind(self, weights):
        n, px = self.names, self.prefix
        # one projection for everything that reads the stream: q | k | v | gate | decay latent
        self.w_in = torch.cat([take_weight(weights, px + n[k]) for k in ("q", "k", "v", "gate", "decay_down")], dim=0).contiguous()
        self.w_decay_up, self.w_out = weights[px + n["decay_up"]], weights[px + n["out"]]
        self.decay_bias, self.norm_w = _f32(weights, px + n["decay_bias"]), _f32(weights, px + n["norm"])

    def kernel_modules(self):
        return ("recurrent", "elementwise", *linear_modules(self.runtime.dtype))

    def state_spec(self):
        return StateSpec((self.heads, self.vdim, self.key_dim), torch.float32)       # column by column

    def forward(self, x, ctx, cache):
        dtype = self.runtime.dtype
        n_qkv = 2 * self.n_qk + self.n_v
        proj = linear(x, self.w_in)
        a_raw = linear(ops.bias_act(proj, None, "none", dtype, n_qkv + self.n_v, self.decay_rank), self.w_decay_up)
        o = ops.gla_scan(proj, a_raw, self.decay_bias, cache.state, ctx, self.heads, self.key_dim, self.vdim, self.q_scale,
                         self.tau, write_state=cache.writable)
        g = ops.gated_part_norm(o, proj, n_qkv, self.norm_w, self.heads, self.eps, gate_first=False, out_dtype=dtype,
                                gate_activation="silu")
        return linear(g, self.w_out)


class GatedDeltaHeadMixer(Mixer):
    """The gated delta rule with ONE decay per head.  q and k (``key_heads`` heads of ``key_dim``) and v (``heads`` heads
    of ``vdim``) each pass a causal convolution (no bias) and SiLU; q and k become unit vectors per head
    (x / sqrt(sum x^2 + ``unit_eps``)), q times key_dim^-1/2; beta = sigmoid(W_b h); g = exp(-exp(A_log_h) *
    softplus(W_a h + dt_bias_h)) per head.  Per head (its q/k head is h // (heads / key_heads)):
    S = g S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q.  Each head's o is RMS-normed over vdim, times a weight
    shared by the heads, times silu(W_g h) (heads x vdim); then the output projection.

    params: hidden_size, heads, key_heads, key_dim, vdim, conv (taps), norm_eps, unit_eps (default 1e-6), names.
    State per sequence: the convolutions' last taps - 1 inputs and S, stored [heads, vdim, key_dim]."""

    NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b",
             "A_log": "A_log", "decay": "a", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "out": "o"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.key_heads = int(p["heads"]), int(p["key_heads"])
        self.key_dim, self.vdim, self.taps = int(p["key_dim"]), int(p["vdim"]), int(p["conv"])
        self.eps, self.unit_eps = float(p["norm_eps"]), float(p.get("unit_eps", 1e-6))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        if self.heads % self.key_heads:
            raise ValueError(f"gated delta rule '{self.prefix}': {self.heads} heads are not a multiple of "
                             f"{self.key_heads} query/key heads")
        for refusal in (conv_taps_refusal(self.taps), state_matrix_refusal(self.key_dim, self.vdim)):
            if refusal:
                raise ValueError(f"gated delta rule '{self.prefix}': {refusal}")
        self.n_qk = self.key_heads * self.key_dim
        self.n_v = self.heads * self.vdim
        self.channels = 2 * self.n_qk + self.n_v

    def tensors(self):
        n, px, D, H = self.names, self.prefix, self.hidden, self.heads
        return [TensorSpec(px + n["q"], (self.n_qk, D), MATRIX), TensorSpec(px + n["q_conv"], (self.n_qk, self.taps), VECTOR),
                TensorSpec(px + n["k"], (self.n_qk, D), MATRIX), TensorSpec(px + n["k_conv"], (self.n_qk, self.taps), VECTOR),
                TensorSpec(px + n["v"], (self.n_v, D), MATRIX), TensorSpec(px + n["v_conv"], (self.n_v, self.taps), VECTOR),
                TensorSpec(px + n["beta"], (H, D), MATRIX), TensorSpec(px + n["A_log"], (H,), VECTOR),
                TensorSpec(px + n["norm"], (self.vdim,), VECTOR, NORM_WEIGHT),
                TensorSpec(px + n["decay"], (H, D), MATRIX), TensorSpec(px + n["dt_bias"], (H,), VECTOR),
                TensorSpec(px + n["gate"], (self.n_v, D), MATRIX), TensorSpec(px + n["out"], (D, self.n_v), MATRIX)]

    def bind(self, weights):
        n, px = self.names, self.prefix
        # one projection for everything that reads the mixer's input: q | k | v | beta | decay | gate
        self.w_in = torch.cat([take_weight(weights, px + n[k]) for k in ("q", "k", "v", "beta", "decay", "gate")], dim=0).contiguous()
        self.conv_w = torch.cat([_f32(weights, px + n[k]) for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.w_out = weights[px + n["out"]]
        self.a_log, self.dt_bias, self.norm_w = (_f32(weights, px + n[k]) for k in ("A_log", "dt_bias", "norm"))

    def kernel_modules(self):
        return ("recurrent", "elementwise", *linear_modules(self.runtime.dtype))

    def state_spec(self):
        state = StateSpec((self.heads, self.vdim, self.key_dim), torch.float32)       # column by column
        return (StateSpec((self.taps - 1, self.channels), torch.float32), state) if self.taps > 1 else state

    def forward(self, x, ctx, cache):
        dtype, C, H = self.runtime.dtype, self.channels, self.heads
        if self.taps > 1:
            tail, state = cache.state
        else:
            tail, state = x.new_zeros((1, 0, C), dtype=torch.float32), cache.state
        proj = linear(x, self.w_in)
        qkv = ops.short_conv(proj, 0, C, self.conv_w, None, tail, ctx, update_tail=cache.writable)
        o = ops.delta_rule(qkv, proj, C, proj, self.dt_bias, self.a_log, state, ctx, H, self.key_heads, self.key_dim,
                           self.vdim, self.unit_eps, self.key_dim ** -0.5, write_state=cache.writable, per_head=True,
                           a_col0=C + H)
        g = ops.gated_part_norm(o, proj, C + 2 * H, self.norm_w, H, self.eps, gate_first=False, out_dtype=dtype,
                                gate_activation="silu")
        return linear(g, self.w_out)


class RetentionMixer(Mixer):
    """Linear attention with a fixed decay per head and neither softmax nor denominator.  q = W_q h and k = W_k h
    (heads x key_dim), v = W_v h (heads x vdim); the position encoding turns the first part of every head of q and k
    (value i with value i + n/2); k times ``k_scale`` after the turn.  Per head S <- decay_h S + k v^T from S = 0 and
    o = S^T q.  Each head's o is divided by its root mean square over vdim (no weight), multiplied by silu(W_g h), and
    projected by W_o.  The turn, the state, the read-out and the norm are 32-bit.

    params: hidden_size, heads, key_dim, vdim, decay (one number per head), norm_eps, k_scale (default key_dim^-1/2),
    names (optional overrides).  ``position``: an encoding that gives cos and sin [T, n/2], or None.
    State per sequence: S, stored [heads, vdim, key_dim]."""

    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o"}

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.key_dim, self.vdim = int(p["heads"]), int(p["key_dim"]), int(p["vdim"])
        self.decays = [float(d) for d in p["decay"]]
        self.eps = float(p["norm_eps"])
        self.k_scale = float(p.get("k_scale", self.key_dim ** -0.5))
        self.names = {**self.NAMES, **dict(p.get("names", {}))}
        self.position = position[0] if isinstance(position, (tuple, list)) else position
        self.rotary_dim = getattr(self.position, "rotary_dim", 0) if self.position is not None else 0
        if len(self.decays) != self.heads:
            raise ValueError(f"retention '{self.prefix}': {len(self.decays)} decays for {self.heads} heads")
        if self.rotary_dim > self.key_dim:
            raise ValueError(f"retention '{self.prefix}': rotary size {self.rotary_dim} exceeds the key size {self.key_dim}")
        refusal = state_matrix_refusal(self.key_dim, self.vdim)
        if refusal:
            raise ValueError(f"retention '{self.prefix}': {refusal}")
        self.n_qk, self.n_v = self.heads * self.key_dim, self.heads * self.vdim

    def tensors(self):
        n, px, D = self.names, self.prefix, self.hidden
        return [TensorSpec(px + n["q"], (self.n_qk, D), MATRIX), TensorSpec(px + n["k"], (self.n_qk, D), MATRIX),
                TensorSpec(px + n["v"], (self.n_v, D), MATRIX), TensorSpec(px + n["gate"], (self.n_v, D), MATRIX),
                TensorSpec(px + n["out"], (D, self.n_v), MATRIX)]

    def bind(self, weights):
        n, px = self.names, self.prefix
        # one projection for everything that reads the mixer's input: q | k | v | gate
        self.w_in = torch.cat([take_weight(weights, px + n[k]) for k in ("q", "k", "v", "gate")], dim=0).contiguous()
        self.w_out = weights[px + n["out"]]
        dev = self.w_out.device
        self.decay = torch.tensor(self.decays, dtype=torch.float32, device=dev)
        self.ones = torch.ones((self.vdim,), dtype=torch.float32, device=dev)

    def kernel_modules(self):
        return ("recurrent", "elementwise", *linear_modules(self.runtime.dtype))

    def state_spec(self):
        return StateSpec((self.heads, self.vdim, self.key_dim), torch.float32)       # column by column

    def forward(self, x, ctx, cache):
        proj = linear(x, self.w_in)
        cos = sin = None
        if self.position is not None and self.rotary_dim:
            cos, sin = self.position.prepare(ctx)
        o = ops.retention_scan(proj, cos, sin, self.rotary_dim, self.decay, cache.state, ctx, self.heads, self.key_dim,
                               self.vdim, 1.0, self.k_scale, write_state=cache.writable)
        g = ops.gated_part_norm(o, proj, 2 * self.n_qk + self.n_v, self.ones, self.heads, self.eps, gate_first=False,
                                out_dtype=self.runtime.dtype, gate_activation="silu")
        return linear(g, self.w_out)


register_mixer("mamba2", Mamba2Mixer)
register_mixer("gated_delta_headwise", GatedDeltaHeadMixer)
register_mixer("retention", RetentionMixer)
register_mixer("rglru", RGLRUMixer)
register_mixer("gated_delta_channelwise", GatedDeltaMixer)
register_mixer("gated_linear_attention", GatedLinearAttentionMixer)
