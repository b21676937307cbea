"""RMS norm: y = v * rsqrt(mean(v^2) + eps) * w, v = x (+ delta), sums in 32-bit
(the reference: core/runtime.cpp:1018-1019, 1066, 1090-1091)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.manifest import NORM_WEIGHT, VECTOR, TensorSpec
from .base import Norm, NormedSum, ScaledSum
from .registry import register_norm


class RMSNorm(Norm):
    """params: dim, eps, name (default "weight"); tensor: <prefix><name> [dim]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.dim = int(spec.params["dim"])
        self.eps = float(spec.params["eps"])
        self.name = self.prefix + str(spec.params.get("name", "weight"))
        self.weight = None

    def tensors(self):
        return [TensorSpec(self.name, (self.dim,), VECTOR, NORM_WEIGHT)]

    def bind(self, weights):
        self.weight = weights[self.name].to(torch.float32).contiguous()

    def kernel_modules(self):
        return ("elementwise",)

    adds_split_sums = True      # ``delta`` may be a SplitSum: the kernel adds its planes
    adds_scaled_sums = True     # ... or a ScaledSum: the kernel multiplies as it adds

    def forward(self, x, delta=None, write_sum=False, rows=None, out_dtype=None):
        if isinstance(delta, ScaledSum):
            return ops.rmsnorm(x, self.weight, self.eps, out_dtype or self.runtime.dtype, delta=delta.y,
                               write_sum=write_sum, rows=rows, delta_scale=delta.scale)
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype or self.runtime.dtype, delta=delta,
                           write_sum=write_sum, rows=rows)

    def add_normed(self, h, y, cast_dtype=None):
        """h += y / rms(y) * w in place (32-bit); the new h in ``cast_dtype`` if one is given."""
        return ops.rmsnorm_onto(h, y, self.weight, self.eps, cast_dtype)

    def norm_sum(self, h, y, alpha=1.0, cast_dtype=None):
        """h <- norm(alpha * h + y) * w in place (32-bit): the norm after the sum; the new h in ``cast_dtype`` if one is
        given."""
        return ops.rmsnorm_mix(h, y, self.weight, self.eps, alpha, cast_dtype)


class LayerNorm(Norm):
    """Layer norm with a weight and no bias: (v - mean) / sqrt(var + eps) * w, var the mean of the squared deviations,
    32-bit.  params: dim, eps, name (default "weight"); tensor: <prefix><name> [dim].  As ``delta`` it also takes a
    ``NormedSum`` of another layer norm: the norm on a sublayer's output, the sum onto the stream and this norm are then
    one kernel."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.dim = int(spec.params["dim"])
        self.eps = float(spec.params["eps"])
        self.name = self.prefix + str(spec.params.get("name", "weight"))
        self.weight = None

    def tensors(self):
        return [TensorSpec(self.name, (self.dim,), VECTOR, NORM_WEIGHT)]

    def bind(self, weights):
        self.weight = weights[self.name].to(torch.float32).contiguous()

    def kernel_modules(self):
        return ("layernorm", "elementwise")

    adds_normed_sums = True

    def forward(self, x, delta=None, write_sum=False, rows=None, out_dtype=None):
        out_dtype = out_dtype or self.runtime.dtype
        if isinstance(delta, NormedSum):
            if write_sum and rows is not None:
                delta.add_onto(x)
                delta = None
            else:
                return ops.layernorm(x, self.weight, self.eps, out_dtype, add=delta.y, add_weight=delta.norm.weight,
                                     add_eps=delta.norm.eps, write_sum=write_sum, rows=rows)
        if delta is not None:
            x = ops.add_inplace(x, delta) if write_sum else x + delta
        return ops.layernorm(x, self.weight, self.eps, out_dtype, rows=rows)

    def add_normed(self, h, y, cast_dtype=None):
        """h += LN(y) * w in place (32-bit); the new h in ``cast_dtype`` if one is given."""
        ops.layernorm(h, None, self.eps, add=y, add_weight=self.weight, write_sum=True)
        if cast_dtype is None:
            return None
        return h if cast_dtype == torch.float32 else ops.bias_act(h, None, "none", cast_dtype)


register_norm("rms", RMSNorm)
register_norm("layer", LayerNorm)
