"""Dense SwiGLU feed-forward: down(up(h) * silu(gate(h))), no biases
(src/llaisys/models/qwen2.cpp:744-759; src/ops/swiglu/op.cpp:17-23, silu as
g / (1 + exp(-g))).  gate and up are one fused product; the activation is
computed in float32 and rounded once; in bfloat16 it is the epilogue of that product."""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import FEED_FORWARDS, FeedForward
from .linear import FusedLinear, GateUpLinear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    takes_deferred = True            # the gate|up product applies the factor

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        names = spec.get("names", {})
        self.gate_up = GateUpLinear(prefix, names.get("gate", "gate_proj"), names.get("up", "up_proj"), self.hidden,
                                    self.intermediate, dtype)
        self.down = FusedLinear(prefix, [names.get("down", "down_proj")], self.intermediate, [self.hidden], False, dtype)

    def params(self) -> List[ParamSpec]:
        return self.gate_up.params() + self.down.params()

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gate_up.bind(tensors)
        self.down.bind(tensors)

    def fused_decode(self):
        if type(self) is not SwiGLU or not self.gate_up.fused_activation or self.down.bias is not None:
            return None
        return {"w_gate_up": self.gate_up.weight, "w_down": self.down.weight, "hidden": self.hidden, "intermediate": self.intermediate}

    def forward(self, h, ctx):
        return self.down(self.gate_up.activation(h))

    def forward_into(self, h, ctx, tail):
        return tail.apply_linear(self.down, self.gate_up.activation(h))


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    """A gated feed-forward with bounded operands: g = min(gate(h), limit), u = clamp(up(h), -limit, limit),
    y = g * sigmoid(alpha * g) * (u + 1), output down(y); no biases.  ``limit`` and ``alpha`` are parameters of the spec.
    gate and up are one product; the activation is computed in float32 and rounded once; in bfloat16 it is the epilogue
    of that product."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        self.limit = float(spec["limit"])
        self.alpha = float(spec.get("alpha", 1.702))
        names = spec.get("names", {})
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        self.gate_up = GateUpLinear(prefix, names.get("gate", "gate_proj"), names.get("up", "up_proj"), self.hidden, self.intermediate, dtype,
                                    suffixes=suffixes, epilogue="glu_clamped", epilogue_params=(self.limit, self.alpha))
        self.down = FusedLinear(prefix, [names.get("down", "down_proj")], self.intermediate, [self.hidden], False, dtype, suffixes=suffixes)

    def params(self) -> List[ParamSpec]:
        return self.gate_up.params() + self.down.params()

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.gate_up.bind(tensors)
        self.down.bind(tensors)

    def forward(self, h, ctx):
        return self.down(self.gate_up.activation(h))


@FEED_FORWARDS.register("polynorm_mlp")
class PolyNormMLP(FeedForward):
    """A dense feed-forward with one inner product and the PolyNorm activation: ``down(act(up(h)))``, both products with
    biases, ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e`` with powers element by element, ``N(v) = v / sqrt(mean(v^2) + eps)``
    over the token's inner vector, and (a, b, c, e) a stored tensor of four numbers.  The three means and the sum are
    float32; the result is rounded once."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        self.eps = float(spec["eps"])
        names = spec.get("names", {})
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        self.up = FusedLinear(prefix, [names.get("up", "up_proj")], self.hidden, [self.intermediate], True, dtype, suffixes=suffixes)
        self.down = FusedLinear(prefix, [names.get("down", "down_proj")], self.intermediate, [self.hidden], True, dtype, suffixes=suffixes)
        self.act_name = prefix + names.get("act", "act")
        self.coef = None

    def params(self) -> List[ParamSpec]:
        return self.up.params() + self.down.params() + [ParamSpec(self.act_name, (4,), role="vector", mean=0.3, std=0.2)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.up.bind(tensors)
        self.down.bind(tensors)
        self.coef = tensors.pop(self.act_name).contiguous()

    def forward(self, h, ctx):
        z = self.up(h)
        act = torch.empty_like(z)
        K.polynorm(z, self.coef, self.eps, act)
        return self.down(act)
