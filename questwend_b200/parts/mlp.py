"""Dense gated feed-forward: down( silu(gate(x)) * up(x) ) (the reference: core/runtime.cpp:1074-1076), with other gates
as parameters: the tanh form of GELU, and a clamped form, g sigmoid(1.702 g) (u + 1) with g = min(gate(x), limit) and
u = up(x) clamped to +-limit."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.manifest import MATRIX, VECTOR, TensorSpec
from .base import FeedForward, take_weight
from .linear import kernel_modules as linear_modules, linear, linear_act, linear_onto, linear_swiglu
from .registry import register_feed_forward


class GatedMLP(FeedForward):
    """params: hidden_size, intermediate_size, activation (on the gate: one of ``ops.GATE_ACTIVATIONS``, default "silu"),
    limit (the bound of "clamped_swish"), names (optional overrides)."""

    NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = str(spec.params.get("activation", "silu"))
        if self.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"feed-forward '{self.prefix}': unknown gate activation '{self.activation}'; known: "
                             f"{', '.join(ops.GATE_ACTIVATIONS)}")
        self.limit = float(spec.params.get("limit", 0.0) or 0.0)
        if self.activation == "clamped_swish" and not self.limit > 0:
            raise ValueError(f"feed-forward '{self.prefix}': the clamped gate needs a positive 'limit', got {self.limit}")
        self.names = {**self.NAMES, **dict(spec.params.get("names", {}))}
        self.w_gate_up = self.w_down = None
        self.interleave = 0

    def tensors(self):
        n, px = self.names, self.prefix
        return [TensorSpec(px + n["gate"], (self.inter, self.hidden), MATRIX),
                TensorSpec(px + n["up"], (self.inter, self.hidden), MATRIX),
                TensorSpec(px + n["down"], (self.hidden, self.inter), MATRIX)]

    def bind(self, weights):
        n, px = self.names, self.prefix
        gate, up = take_weight(weights, px + n["gate"]), take_weight(weights, px + n["up"])      # only copied from
        # one fused projection.  Where the sizes allow, gate and up rows are interleaved in groups of 8 features, so that the
        # products with a fused SwiGLU epilogue find both in one thread (a reordering of rows: the same numbers).
        self.interleave = ops.GATE_UP_GROUP if self.inter % ops.GATE_UP_GROUP == 0 else 0
        if self.interleave:
            self.w_gate_up = ops.interleave_gate_up(gate, up, self.interleave)
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        del gate, up
        self.w_down = weights[px + n["down"]]

    def kernel_modules(self):
        return ("elementwise", *linear_modules(self.runtime.dtype))

    adds_to_residual = True

    def forward(self, x, ctx, residual=None):
        act = linear_swiglu(x, self.w_gate_up, self.runtime.dtype, self.interleave, self.activation, self.limit)
        if residual is not None:
            return linear_onto(act, self.w_down, residual)  # None: the residual sum was made in the product's epilogue
        return linear(act, self.w_down)


class BiasedMLP(FeedForward):
    """Ungated: down( act(up(x) + b_up) ) + b_down, or without the biases: down(act(up(x))).
    params: hidden_size, intermediate_size, activation (one of ``ops.ACTIVATIONS``; one with learned numbers of its own,
    as "xielu" has, reads them from the tensor ``act``), biases (default True), names (optional overrides)."""

    NAMES = {"up": "up", "up_bias": "up.b", "down": "down", "down_bias": "down.b", "act": "act"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = str(spec.params["activation"])
        self.biases = bool(spec.params.get("biases", True))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"feed-forward '{self.prefix}': unknown activation '{self.activation}'; known: "
                             f"{', '.join(ops.ACTIVATIONS)}")
        self.n_act_params = ops.ACTIVATION_PARAMS.get(self.activation, 0)
        self.names = {**self.NAMES, **dict(spec.params.get("names", {}))}
        self.b_up = self.b_down = self.act_params = None

    def tensors(self):
        n, px = self.names, self.prefix
        out = [TensorSpec(px + n["up"], (self.inter, self.hidden), MATRIX), TensorSpec(px + n["up_bias"], (self.inter,), VECTOR),
               TensorSpec(px + n["down"], (self.hidden, self.inter), MATRIX), TensorSpec(px + n["down_bias"], (self.hidden,), VECTOR)]
        if not self.biases:
            out = [out[0], out[2]]
        if self.n_act_params:
            out.append(TensorSpec(px + n["act"], (self.n_act_params,), VECTOR))
        return out

    def bind(self, weights):
        n, px = self.names, self.prefix
        self.w_up, self.w_down = weights[px + n["up"]], weights[px + n["down"]]
        if self.biases:
            self.b_up = weights[px + n["up_bias"]].to(torch.float32).contiguous()
            self.b_down = weights[px + n["down_bias"]].to(torch.float32).contiguous()
        if self.n_act_params:
            self.act_params = weights[px + n["act"]].to(torch.float32).contiguous()

    def kernel_modules(self):
        return ("elementwise", *linear_modules(self.runtime.dtype))

    def forward(self, x, ctx):
        act = linear_act(x, self.w_up, self.b_up, self.activation, self.runtime.dtype, params=self.act_params)
        out = linear(act, self.w_down)
        return ops.bias_act(out, self.b_down, "none", torch.float32) if self.biases else out


register_feed_forward("gated_mlp", GatedMLP)
register_feed_forward("biased_mlp", BiasedMLP)
register_feed_forward("plain_mlp", BiasedMLP)        # the same part under the name a plan without biases reads better with
