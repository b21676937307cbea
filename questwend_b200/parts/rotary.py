"""Rotary position encoding, NeoX form: the pairs (i, i + n_rot/2) of a head are rotated by
pos * theta^(-2i/n_rot); dims from n_rot on pass through (the reference: core/runtime.cpp:300-301,
ggml-cpu/ops.cpp:5934-5950).  The inverse frequencies are made once in float64; each step's
cos/sin table is made once and shared by every layer that uses this encoding."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import PositionEncoding
from .registry import register_position


class RotaryEncoding(PositionEncoding):
    """params: theta, rotary_dim, linear_factor (every frequency is divided by it: positions shrink by that factor;
    default 1)."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary size {self.rotary_dim} must be positive and even")
        self.linear_factor = float(spec.params.get("linear_factor", 1.0) or 1.0)
        if not self.linear_factor > 0:
            raise ValueError(f"rotary scaling factor {self.linear_factor} must be positive")
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-2.0 * i / self.rotary_dim) / self.linear_factor).to(runtime.device)

    def kernel_modules(self):
        return ("rope_kv",)

    def prepare(self, ctx):
        key = ("rotary", id(self))
        if key not in ctx.shared:
            ctx.shared[key] = ops.rope_table(ctx.tok_pos, self.inv_freq)
        return ctx.shared[key]


def scaled_frequencies(rotary_dim: int, theta: float, factor=None, original=None, fast=None, slow=None):
    """Angle per position of each pair, in float64, and the factor on cos and sin.  Without ``factor``: theta^(-2i/n), 1.
    With it (the YaRN form): let d(r) = n ln(original / (2 pi r)) / (2 ln theta), lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), n - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); pair i turns by
    f_i / factor * ramp_i + f_i * (1 - ramp_i), and cos and sin are multiplied by 0.1 ln(factor) + 1."""
    import math
    n = rotary_dim
    i = torch.arange(n // 2, dtype=torch.float64)
    f = theta ** (-2.0 * i / n)
    if factor is None:
        return f, 1.0

    def pair_of(turns):
        return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), n - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class PairedRotaryEncoding(PositionEncoding):
    """Rotation of neighbouring pairs (2i, 2i + 1) of the first ``rotary_dim`` values, optionally scaled for long
    contexts.  params: theta, rotary_dim, and for the scaling (all four or none) factor, original, fast, slow.
    ``prepare`` gives cos and sin [T, rotary_dim / 2] with the scaling's factor already on them; which values are
    paired is the business of the kernel that applies them."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.theta = float(p["theta"])
        self.rotary_dim = int(p["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary size {self.rotary_dim} must be positive and even")
        scaling = [p.get(k) for k in ("factor", "original", "fast", "slow")]
        if any(v is None for v in scaling) and not all(v is None for v in scaling):
            raise ValueError("a scaled rotation needs all of factor, original, fast and slow")
        freqs, self.factor = scaled_frequencies(self.rotary_dim, self.theta, *[None if v is None else float(v) for v in scaling])
        self.inv_freq = freqs.to(runtime.device)

    def kernel_modules(self):
        return ("rope_kv",)

    def prepare(self, ctx):
        key = ("rotary_pairs", id(self))
        if key not in ctx.shared:
            ctx.shared[key] = ops.rope_table(ctx.tok_pos, self.inv_freq, self.factor)
        return ctx.shared[key]


def wavelength_scaled_frequencies(rotary_dim: int, theta: float, factor: float, low: float, high: float, original: float):
    """Angle per position of each pair, in float64, scaled by wavelength: with f_i = theta^(-2i/n) and wavelength
    l = 2 pi / f, a pair keeps f where l < original / high, turns by f / factor where l > original / low, and between the
    two by (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    import math
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = theta ** (-2.0 * i / rotary_dim)
    wavelength = 2.0 * math.pi / f
    s = (original / wavelength - low) / (high - low)
    mixed = (1.0 - s) * f / factor + s * f
    return torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, mixed))


class WavelengthScaledRotary(PositionEncoding):
    """Rotation angles theta^(-2i/n), optionally scaled by wavelength for contexts longer than the ``original`` one.
    params: theta, rotary_dim, and for the scaling (all four or none) factor, low, high, original.  ``prepare`` gives cos
    and sin [T, rotary_dim / 2]; which values are paired is the business of the kernel that applies them."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.theta = float(p["theta"])
        self.rotary_dim = int(p["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary size {self.rotary_dim} must be positive and even")
        scaling = [p.get(k) for k in ("factor", "low", "high", "original")]
        if any(v is None for v in scaling) and not all(v is None for v in scaling):
            raise ValueError("a rotation scaled by wavelength needs all of factor, low, high and original")
        if scaling[0] is None:
            i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            freqs = self.theta ** (-2.0 * i / self.rotary_dim)
        else:
            freqs = wavelength_scaled_frequencies(self.rotary_dim, self.theta, *[float(v) for v in scaling])
        self.inv_freq = freqs.to(runtime.device)

    def kernel_modules(self):
        return ("rope_kv",)

    def prepare(self, ctx):
        key = ("rotary_wavelength", id(self))
        if key not in ctx.shared:
            ctx.shared[key] = ops.rope_table(ctx.tok_pos, self.inv_freq)
        return ctx.shared[key]


register_position("rotary_neox", RotaryEncoding)
register_position("rotary_pairs", PairedRotaryEncoding)
register_position("rotary_wavelength", WavelengthScaledRotary)
