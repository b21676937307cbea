"""Mixers made of other mixers.  ``SideBySideMixer``: several mixers read the same input side by side; the output is the
sum of theirs, each times a constant, optionally each RMS-normed first.  ``InputConvMixer``: a short causal convolution
over time in front of any mixer.  The inner mixers are ordinary registered ones (attention, a recurrence, ...): each
keeps what it keeps (paged keys and values, fixed-size state), and these parts hand every one its share of the layer's
cache unit."""
from __future__ import annotations

from dataclasses import replace

import torch

from ..kernels import ops
from ..kernels.limits import conv_taps_refusal
from ..weights.manifest import NORM_WEIGHT, VECTOR, TensorSpec
from .base import KVSpec, Mixer, PartSpec, StateSpec, UnitCache
from .registry import build_part, register_mixer


def _as_tuple(spec, single_type):
    if spec is None:
        return ()
    return (spec,) if isinstance(spec, single_type) else tuple(spec)


class SideBySideMixer(Mixer):
    """params: branches, a list of {"name": tensor-name stem under this mixer's prefix, "spec": PartSpec of a mixer,
    "scale": constant on its output (default 1), "norm": None or {"name": tensor name under this mixer's prefix, "dim",
    "eps"}: the branch's output is RMS-normed over its row with that weight before it is scaled and added}.
    ``position``: one encoding per branch (or None), in the same order.
    The cache unit of the layer holds the branches' key/value groups and states one after the other."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        branches = list(spec.params["branches"])
        if not branches:
            raise ValueError(f"mixer '{self.prefix}': no branches")
        positions = list(position) if isinstance(position, (tuple, list)) else [position] + [None] * (len(branches) - 1)
        if len(positions) != len(branches):
            raise ValueError(f"mixer '{self.prefix}': {len(positions)} position encodings for {len(branches)} branches")
        self.branches, self.scales, self.norms = [], [], []
        for b, pos in zip(branches, positions):
            sub: PartSpec = b["spec"]
            self.branches.append(build_part("mixer", replace(sub, prefix=self.prefix + str(b["name"]) + "."), runtime, position=pos))
            self.scales.append(float(b.get("scale", 1.0)))
            n = b.get("norm")
            self.norms.append(None if n is None else (self.prefix + str(n["name"]), int(n["dim"]), float(n["eps"])))
        self.norm_w = [None] * len(self.branches)
        self._kv = [_as_tuple(m.kv_spec(), KVSpec) for m in self.branches]
        self._state = [_as_tuple(m.state_spec(), StateSpec) for m in self.branches]
        self._state_single = [isinstance(m.state_spec(), StateSpec) for m in self.branches]

    def tensors(self):
        out = [t for m in self.branches for t in m.tensors()]
        return out + [TensorSpec(n[0], (n[1],), VECTOR, NORM_WEIGHT) for n in self.norms if n is not None]

    def bind(self, weights):
        for m in self.branches:
            m.bind(weights)
        for i, n in enumerate(self.norms):          # the branch's constant rides on its norm's weight
            if n is not None:
                self.norm_w[i] = (weights[n[0]].to(torch.float32) * self.scales[i]).contiguous()

    def kernel_modules(self):
        return ("elementwise", *(k for m in self.branches for k in m.kernel_modules()))

    def kv_spec(self):
        flat = tuple(s for group in self._kv for s in group)
        return None if not flat else (flat[0] if len(flat) == 1 else flat)

    def state_spec(self):
        flat = tuple(s for group in self._state for s in group)
        return None if not flat else (flat[0] if len(flat) == 1 else flat)

    def _share(self, cache: UnitCache, i: int) -> UnitCache:
        """Branch i's part of the layer's cache unit."""
        n_kv = sum(len(g) for g in self._kv)
        views = [] if not n_kv else [cache, *cache.more]
        states = () if cache.state is None else (cache.state if isinstance(cache.state, tuple) else (cache.state,))
        k0, s0 = sum(len(g) for g in self._kv[:i]), sum(len(g) for g in self._state[:i])
        mine = views[k0:k0 + len(self._kv[i])]
        st = states[s0:s0 + len(self._state[i])]
        state = None if not st else (st[0] if self._state_single[i] else tuple(st))
        if not mine:
            return UnitCache(None, None, None, state, cache.writable)
        first = mine[0]
        return UnitCache(first.group_id, first.k_pool, first.v_pool, state, cache.writable, more=tuple(mine[1:]))

    def forward(self, x, ctx, cache):
        out = None
        for i, (m, scale) in enumerate(zip(self.branches, self.scales)):
            y = m.forward(x, ctx, self._share(cache, i))
            if self.norms[i] is not None:
                if out is None:
                    out = ops.rmsnorm(y, self.norm_w[i], self.norms[i][2], torch.float32)
                else:
                    ops.rmsnorm_onto(out, y, self.norm_w[i], self.norms[i][2])
            else:
                out = ops.scale_softcap(y, scale, 0.0) if out is None else ops.add_inplace(out, y, scale)
        return out


class InputConvMixer(Mixer):
    """What the inner mixer reads is x + conv(x): a causal convolution over time on every channel of the mixer's input,
    conv(x)_t = sum_j w[:, j] x_(t - taps + 1 + j), zeros before the sequence's start, no bias, no activation.  The
    convolution runs in 32-bit on the 32-bit stream (``reads_stream``) and hands the inner mixer its input in the engine's
    dtype; its last taps - 1 inputs are per-sequence state, in front of the inner mixer's own in the layer's cache unit.
    params: inner (PartSpec of a mixer; it gets this mixer's prefix), channels, taps, weight (the FULL name of the tensor
    [channels, taps]: it need not lie under this mixer's prefix).  ``position`` goes to the inner mixer."""

    reads_stream = True

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.channels, self.taps = int(p["channels"]), int(p["taps"])
        self.weight_name = str(p["weight"])
        refusal = conv_taps_refusal(self.taps)
        if refusal:
            raise ValueError(f"mixer '{self.prefix}': {refusal}")
        self.inner = build_part("mixer", replace(p["inner"], prefix=self.prefix), runtime, position=position)
        self._inner_single = isinstance(self.inner.state_spec(), StateSpec)
        self.conv_w = None

    def tensors(self):
        return [TensorSpec(self.weight_name, (self.channels, self.taps), VECTOR), *self.inner.tensors()]

    def bind(self, weights):
        self.conv_w = weights[self.weight_name].to(torch.float32).contiguous()
        self.inner.bind(weights)

    def kernel_modules(self):
        return ("recurrent", *self.inner.kernel_modules())

    def kv_spec(self):
        return self.inner.kv_spec()

    def state_spec(self):
        mine = (StateSpec((self.taps - 1, self.channels), torch.float32),) if self.taps > 1 else ()
        flat = mine + _as_tuple(self.inner.state_spec(), StateSpec)
        return None if not flat else (flat[0] if len(flat) == 1 else flat)

    def forward(self, x, ctx, cache):
        states = () if cache.state is None else (cache.state if isinstance(cache.state, tuple) else (cache.state,))
        if self.taps > 1:
            tail, rest = states[0], states[1:]
        else:
            tail, rest = x.new_zeros((1, 0, self.channels), dtype=torch.float32), states
        if x.dtype != torch.float32:                # a block that handed out the stream's copy instead of the stream
            x = x.to(torch.float32)
        y = ops.short_conv(x, 0, self.channels, self.conv_w, None, tail, ctx, activation=False, update_tail=cache.writable,
                           plus_input=True, out_dtype=self.runtime.dtype)
        state = None if not rest else (rest[0] if self._inner_single else tuple(rest))
        inner = UnitCache(cache.group_id, cache.k_pool, cache.v_pool, state, cache.writable, more=cache.more)
        return self.inner.forward(y, ctx, inner)


register_mixer("side_by_side", SideBySideMixer)
register_mixer("input_conv", InputConvMixer)
