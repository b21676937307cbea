"""A mixer made of several mixers that read the same input side by side; its output is the sum of theirs, each times a
constant.  The branches are ordinary registered mixers (attention, a recurrence, ...): each keeps what it keeps
(paged keys and values, fixed-size state), and this part hands every branch its share of the layer's cache unit."""
from __future__ import annotations

from dataclasses import replace

from ..kernels import ops
from .base import KVSpec, Mixer, PartSpec, StateSpec, UnitCache
from .registry import build_part, register_mixer


def _as_tuple(spec, single_type):
    if spec is None:
        return ()
    return (spec,) if isinstance(spec, single_type) else tuple(spec)


class SideBySideMixer(Mixer):
    """params: branches, a list of {"name": tensor-name stem under this mixer's prefix, "spec": PartSpec of a mixer,
    "scale": constant on its output (default 1)}.  ``position``: one encoding per branch (or None), in the same order.
    The cache unit of the layer holds the branches' key/value groups and states one after the other."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        branches = list(spec.params["branches"])
        if not branches:
            raise ValueError(f"mixer '{self.prefix}': no branches")
        positions = list(position) if isinstance(position, (tuple, list)) else [position] + [None] * (len(branches) - 1)
        if len(positions) != len(branches):
            raise ValueError(f"mixer '{self.prefix}': {len(positions)} position encodings for {len(branches)} branches")
        self.branches, self.scales = [], []
        for b, pos in zip(branches, positions):
            sub: PartSpec = b["spec"]
            self.branches.append(build_part("mixer", replace(sub, prefix=self.prefix + str(b["name"]) + "."), runtime, position=pos))
            self.scales.append(float(b.get("scale", 1.0)))
        self._kv = [_as_tuple(m.kv_spec(), KVSpec) for m in self.branches]
        self._state = [_as_tuple(m.state_spec(), StateSpec) for m in self.branches]
        self._state_single = [isinstance(m.state_spec(), StateSpec) for m in self.branches]

    def tensors(self):
        return [t for m in self.branches for t in m.tensors()]

    def bind(self, weights):
        for m in self.branches:
            m.bind(weights)

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
            out = ops.scale_softcap(y, scale, 0.0) if out is None else ops.add_inplace(out, y, scale)
        return out


register_mixer("side_by_side", SideBySideMixer)
