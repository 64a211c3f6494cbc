"""A mixture of experts: many small gated feed-forward layers, of which each token uses a few.

    z = W_router h                      (float32 logits)
    s = sigmoid(z)                      the scores; the ``top`` largest choose a token's experts (``scoring``: sigmoid)
    w_e = s_e                           their weights: the scores as they are (``renormalize``: divided by their sum)
    y = sum_e expert_e(w_e h)           ``weight_on`` "input"; or  y = sum_e w_e expert_e(h)  with "output"
    expert(u) = W_down (silu(W_gate u) * (W_up u)), no biases.

``scoring`` "softmax_chosen": the ``top`` largest logits choose a token's experts, and the weights are the softmax over
the chosen logits alone.  ``router_bias`` true: ``z = W_router h + b``.

``scoring`` "softmax_grouped": the router has ``experts + identity`` outputs; ``s = softmax(z)`` over all of them; the
choice scores are ``s + correction`` (a stored vector); the outputs form ``groups`` equal groups of neighbours, a group's
score is its largest choice score, and only outputs of the ``keep_groups`` best groups can be chosen; the ``top`` largest
choice scores choose; the weights are the chosen outputs' s divided by their sum (+ 1e-20), times ``route_scale``.  The last
``identity`` outputs are identity experts: they have no tensors and their output is the input h itself (times the weight).
``activation`` "glu_clamped" (with ``limit``, ``alpha``): ``g = min(W_gate u, limit)``, ``up = clamp(W_up u, -limit, limit)``,
the expert's inner activation is ``g sigmoid(alpha g) (up + 1)`` instead of ``silu(gate) up``.

How a step runs it: the router's product with a float32 result, the choice per token (one warp a token), a stable
counting sort of the (token, choice) pairs by expert on the device (in a step of many tokens every expert's run starts
at a multiple of 128 rows), one gather that builds the experts' input rows in sorted order (with the weight on them), a product per expert over its run of rows for gate|up and for down
(``kernels.grouped_linear`` with the row offsets the sort left on the device), and a combine that sums a token's rows in
the order of its choices (a kernel of its own, or part of the kernel that adds the result to the residual stream).  Nothing comes back to the host, so the launches are the same whatever the routing, and a step
of single tokens can be captured.  A row's result does not depend on which rows share its expert.
Identity experts take part in the sort like the others, behind them: their gathered rows are the input rows, no product
touches them (they belong to no group of the products), and the combine takes them as they are.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import FEED_FORWARDS, FeedForward
from .linear import FusedLinear


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    PAD = 128                      # rows of a tensor-core tile
    PAD_FROM_ROWS = 256            # (token, choice) pairs of a step from which the runs are padded

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.intermediate = int(spec["intermediate_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        if not 0 < self.top <= self.experts + int(spec.get("identity") or 0):
            raise ValueError(f"{self.top} of {self.experts} experts")
        self.scoring = str(spec.get("scoring", "sigmoid"))
        if self.scoring not in ("sigmoid", "softmax_chosen", "softmax_grouped"):
            raise ValueError(f"routing by '{spec.get('scoring')}' is not supported (sigmoid, softmax_chosen, softmax_grouped)")
        self.renormalize = bool(spec.get("renormalize", False))
        if self.renormalize and self.scoring != "softmax_grouped":
            raise ValueError("renormalised routing weights are not supported")
        self.weight_on = str(spec.get("weight_on", "output"))
        if self.weight_on not in ("input", "output"):
            raise ValueError(f"weight_on must be 'input' or 'output', got {self.weight_on!r}")
        # identity experts: router outputs behind the experts' that stand for the input itself
        self.identity = int(spec.get("identity") or 0)
        self.outputs = self.experts + self.identity
        self.groups = int(spec.get("groups") or 1)
        self.keep_groups = int(spec.get("keep_groups") or self.groups)
        self.route_scale = float(spec.get("route_scale", 1.0))
        if self.scoring != "softmax_grouped" and (self.identity or self.groups != 1):
            raise ValueError("identity experts and groups of experts go with scoring 'softmax_grouped'")
        if self.identity and self.weight_on != "output":
            raise ValueError("identity experts take their weight on the output")
        if self.scoring == "softmax_grouped":
            if self.top > self.outputs or self.outputs % self.groups or not 1 <= self.keep_groups <= self.groups or \
                    self.keep_groups * (self.outputs // self.groups) < self.top:
                raise ValueError(f"{self.keep_groups} of {self.groups} groups over {self.outputs} router outputs cannot give {self.top} choices")
        self.activation = str(spec.get("activation", "swiglu"))
        if self.activation not in ("swiglu", "glu_clamped"):
            raise ValueError(f"expert activation {self.activation!r} is not supported (swiglu, glu_clamped)")
        self.limit, self.alpha = float(spec.get("limit", 0.0)), float(spec.get("alpha", 1.702))
        n = dict(spec.get("names", {}))
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        self.router = FusedLinear(prefix, [n.get("router", "gate")], self.hidden, [self.outputs], bool(spec.get("router_bias", False)), dtype,
                                  suffixes=suffixes)
        self.correction_name = prefix + n.get("correction", "correction") if self.scoring == "softmax_grouped" else None
        self.correction = None
        stem = n.get("expert", "experts.{}.")                 # the e-th expert's tensors start with prefix + stem.format(e)
        w = suffixes[0]
        self.expert_names = [tuple(prefix + stem.format(e) + n.get(k, d) + w for k, d in (("gate", "gate_proj"), ("up", "up_proj"), ("down", "down_proj")))
                             for e in range(self.experts)]
        self.gate_up = self.down = None                       # [E, 2 F, hidden] (gate rows, then up rows) and [E, hidden, F]
        # bfloat16 with sizes that are multiples of 8: gate and up rows of every expert interleaved in eights when bound, and
        # the gated activation is the epilogue of the grouped product (the [rows, 2 F] product never goes to memory)
        self.fused_activation = dtype == torch.bfloat16 and self.intermediate % 8 == 0 and self.hidden % 8 == 0
        self.activation_params = None                        # (limit, alpha) on the device, for the epilogue

    def params(self) -> List[ParamSpec]:
        out = self.router.params()
        if self.correction_name:
            out.append(ParamSpec(self.correction_name, (self.outputs,), role="vector", std=0.02))
        F, W = self.intermediate, self.hidden
        for g, u, d in self.expert_names:
            out += [ParamSpec(g, (F, W), role="matrix"), ParamSpec(u, (F, W), role="matrix"), ParamSpec(d, (W, F), role="matrix")]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.router.bind(tensors)
        if self.correction_name:
            self.correction = tensors.pop(self.correction_name)
        gu, dn = [], []
        for g, u, d in self.expert_names:
            gate, up = tensors.pop(g), tensors.pop(u)
            gu.append(K.interleave_gate_up(gate, up) if self.fused_activation else torch.cat([gate, up], dim=0))
            dn.append(tensors.pop(d))
        self.gate_up = torch.stack(gu).contiguous()
        self.down = torch.stack(dn).contiguous()
        if self.activation == "glu_clamped":
            self.activation_params = torch.tensor([self.limit, self.alpha], dtype=torch.float32, device=self.down.device)

    # forward_rows: the experts' output rows and where each token's lie (kernels.RowSum), for a block whose next kernel takes
    # the sum in (parts.block.SandwichBlock); forward: the sum itself
    produces_row_sums = True

    def forward(self, h, ctx):
        return self.forward_rows(h, ctx).materialize()

    def forward_rows(self, h, ctx) -> "K.RowSum":
        T = h.shape[0]
        E, top, F = self.experts, self.top, self.intermediate
        n_out = self.outputs                                   # experts and identity experts: what the router chooses among
        dev = h.device
        logits = self.router(h, out_dtype=torch.float32)
        ids = torch.empty((T, top), dtype=torch.int32, device=dev)
        weights = torch.empty((T, top), dtype=torch.float32, device=dev)
        if self.scoring == "softmax_grouped":
            K.moe_route_grouped(logits, self.correction, top, self.groups, self.keep_groups, self.route_scale, ids, weights)
        else:
            K.moe_route(logits, top, ids, weights, scoring=self.scoring)
        # a step of many tokens: every expert's run of rows starts at a multiple of 128, so that the products run on
        # tensor-core tiles of 128 rows, each of one expert
        pad = self.PAD if (self.dtype == torch.bfloat16 and T * top >= self.PAD_FROM_ROWS) else 1
        R = K.sorted_rows(T * top, n_out, pad)
        offsets = torch.empty(n_out + 1, dtype=torch.int32, device=dev)
        pair_at = torch.empty(R, dtype=torch.int32, device=dev)
        place_of = torch.empty(T * top, dtype=torch.int32, device=dev)
        tiles = torch.empty(R // pad, dtype=torch.int32, device=dev) if pad > 1 else None
        K.moe_sort(ids, n_out, offsets, pair_at, place_of, pad, tiles, matrices=E)
        # (the products see the experts' runs only: the identity experts' rows, behind them, stay as the gather made them)
        expert_offsets = offsets[:E + 1] if n_out != E else offsets
        on_input = self.weight_on == "input"
        rows = torch.empty((R, self.hidden), dtype=self.dtype, device=dev)
        K.moe_gather(h, pair_at, weights if on_input else None, top, rows)
        act = torch.empty((R, F), dtype=self.dtype, device=dev)
        if self.fused_activation:
            K.grouped_linear(rows, self.gate_up, act, expert_offsets, tile_group=tiles, epilogue=self.activation,
                             epilogue_params=self.activation_params)
        else:
            both = torch.empty((R, 2 * F), dtype=self.dtype, device=dev)
            K.grouped_linear(rows, self.gate_up, both, expert_offsets, tile_group=tiles)
            if self.activation == "swiglu":
                K.swiglu(both, act)
            else:
                K.glu_clamped(both, act, self.limit, self.alpha)
        K.grouped_linear(act, self.down, rows, expert_offsets, tile_group=tiles)
        return K.RowSum(rows, place_of, top, None if on_input else weights)
