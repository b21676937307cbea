"""A model built from a plan: embedding, the layers' blocks, final norm, output head.

``forward`` runs one step's packed tokens through the schedule and returns the
logits at the wanted rows only (the reference computes logits for every row of
a prompt and keeps the last, core/runtime.cpp:1093-1095, 3179-3183).
"""
from __future__ import annotations

import torch

from ..parts.base import BoundWeights, Runtime, StepContext, UnitCache
from ..parts.linear import settle
from ..parts.registry import build_part
from ..weights.manifest import TensorSpec
from .plan import ModelPlan


class Model:
    def __init__(self, plan: ModelPlan, runtime: Runtime):
        plan.validate()
        self.plan = plan
        self.runtime = runtime
        self.embedding = build_part("embedding", plan.embedding, runtime)
        self._positions: dict = {}
        self.blocks = []
        for layer in plan.layers:
            position = None
            if isinstance(layer.position, (tuple, list)):       # a mixer that turns several things (keys, values)
                position = tuple(None if spec is None else self._position(spec) for spec in layer.position)
            elif layer.position is not None:
                position = self._position(layer.position)
            self.blocks.append(build_part("block", layer.block, runtime, layer=layer, position=position))
        self.final_norm = build_part("norm", plan.final_norm, runtime)
        self.head = build_part("head", plan.head, runtime)
        self.schedule = list(plan.schedule)
        self.before = [None if run.before is None else build_part("stream_step", run.before, runtime) for run in self.schedule]

    def _position(self, spec):
        key = (spec.kind, tuple(sorted(spec.params.items())))
        if key not in self._positions:                  # layers with the same encoding share one object
            self._positions[key] = build_part("position", spec, self.runtime)
        return self._positions[key]

    # ---- weights
    def parts(self):
        return [self.embedding, *self.blocks, *(b for b in self.before if b is not None), self.final_norm, self.head]

    def tensors(self) -> list[TensorSpec]:
        seen, out = set(), []
        for part in self.parts():
            for t in part.tensors():
                if t.name not in seen:
                    seen.add(t.name)
                    out.append(t)
        return out

    def bind(self, weights: dict) -> None:
        """Hand every part its tensors.  Tensors that a part only copies from (into a fused matrix) are taken out of
        ``weights`` as the binding goes, unless another part names them too."""
        uses: dict = {}
        for part in self.parts():
            for t in part.tensors():
                uses[t.name] = uses.get(t.name, 0) + 1
        bound = BoundWeights(weights, uses)
        for part in self.parts():
            part.bind(bound)

    def kernel_modules(self) -> list[str]:
        mods = []
        for part in self.parts() + list(self._positions.values()):
            for m in part.kernel_modules():
                if m not in mods:
                    mods.append(m)
        return mods

    # ---- cache needs, one entry per scheduled run
    def cache_units(self):
        """[(kv_spec or None, state_spec or None, cache_of or None)] in schedule order."""
        out = []
        for run in self.schedule:
            mixer = self.blocks[run.layer].mixer
            out.append((mixer.kv_spec(), mixer.state_spec(), run.cache_of))
        return out

    # ---- one step
    def forward(self, ctx: StepContext, unit_caches: list[UnitCache], want_rows: torch.Tensor, tap=None) -> torch.Tensor:
        """``tap(run index, stream)``, if given, is called after every scheduled run with the residual stream as it
        stands there (what is still to be added is added first: slower, for looking at a model layer by layer)."""
        for position in self._positions.values():       # the step's tables first: no layer's kernels find them half made
            position.prepare(ctx)
        h = self.embedding.forward(ctx.token_ids)
        delta = None
        for i, run in enumerate(self.schedule):
            if self.before[i] is not None:              # adds onto the stream; what is pending in ``delta`` stays pending
                self.before[i].forward(h, ctx)
            h, delta = self.blocks[run.layer].forward(h, delta, ctx, unit_caches[i])
            if tap is not None:
                if delta is not None:
                    if hasattr(delta, "add_onto"):
                        delta.add_onto(h)
                    else:
                        h.add_(delta)
                    delta = None
                tap(i, h)
        if want_rows.numel() == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=h.device)
        x = self.final_norm.forward(h, settle(h, delta, self.final_norm), rows=want_rows)
        return self.head.forward(x)
