"""Selective state-space mixer (the scalar-decay form with heads and groups).

With inner = heads * head_dim, N = state_size, G = groups, one product of the input gives
``[z: inner | x: inner | B: G N | C: G N | dt: heads]``.  x, B and C together pass a causal convolution per
channel over the last ``conv`` inputs (weights ``[channels, conv]``, the last column the current token's, a bias,
zeros before the first token) and silu.  ``dt = softplus(dt + dt_bias)``.  Per head (head h uses group
``h // (heads / G)``), with S of size N x head_dim and zeros before the first token:

    S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T,        y_t = S_t^T C_t + D_h x_t.

y (heads side by side) is multiplied by silu(z), RMS-normalised in ``norm_groups`` equal parts, multiplied by a
weight, and mapped out.  Step sizes, decays, the state and every sum of the recurrence and of the norm are
float32.  A request's state slot holds S of every head and, behind it, the last ``conv - 1`` inputs of the
convolution; both move on by whatever the step holds of the request.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import MIXERS, FixedState, Mixer
from .linear import FusedLinear
from .scan import scan_chunks


@MIXERS.register("selective_ssm")
class SelectiveStateSpace(Mixer):
    decodes_from_device = True

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.head_dim = int(spec["head_dim"])
        self.state_size = int(spec["state_size"])
        self.groups = int(spec.get("groups", 1))
        self.taps = int(spec["conv"])
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.eps = float(spec["eps"])
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.groups} groups")
        self.inner = self.heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ValueError(f"an inner width of {self.inner} does not split into {self.norm_groups} norm groups")
        self.channels = self.inner + 2 * self.groups * self.state_size
        n = dict(spec.get("names", {}))
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        self.inp = FusedLinear(prefix, [n.get("in", "in_proj")], self.hidden, [2 * self.inner + 2 * self.groups * self.state_size + self.heads],
                               False, dtype, suffixes=suffixes)
        self.out = FusedLinear(prefix, [n.get("o", "out_proj")], self.inner, [self.hidden], False, dtype, suffixes=suffixes)
        self.names = {k: prefix + n.get(k, d) for k, d in (("conv", "conv1d.weight"), ("conv_bias", "conv1d.bias"), ("dt_bias", "dt_bias"),
                                                           ("A_log", "A_log"), ("D", "D"), ("norm", "norm.weight"))}
        self.conv_w = self.conv_b = self.dt_bias = self.A_log = self.D = self.norm_weight = None
        self.scan_elements = self.heads * self.state_size * self.head_dim

    def params(self) -> List[ParamSpec]:
        nm = self.names
        return self.inp.params() + self.out.params() + [
            ParamSpec(nm["conv"], (self.channels, self.taps), role="vector", std=0.3),
            ParamSpec(nm["conv_bias"], (self.channels,), role="vector", std=0.1),
            ParamSpec(nm["dt_bias"], (self.heads,), role="vector", std=0.5),
            ParamSpec(nm["A_log"], (self.heads,), role="vector", std=0.5),
            ParamSpec(nm["D"], (self.heads,), role="vector", init="ones_normal"),
            ParamSpec(nm["norm"], (self.inner,), role="vector", init="ones_normal"),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.inp.bind(tensors)
        self.out.bind(tensors)
        nm = self.names
        self.conv_w, self.conv_b = tensors.pop(nm["conv"]), tensors.pop(nm["conv_bias"])
        self.dt_bias, self.A_log, self.D = tensors.pop(nm["dt_bias"]), tensors.pop(nm["A_log"]), tensors.pop(nm["D"])
        self.norm_weight = tensors.pop(nm["norm"])

    def cache_requirement(self):
        return FixedState((self.scan_elements + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, h, ctx, cache):
        T = h.shape[0]
        proj = self.inp(h)
        xbc = torch.empty((T, self.channels), dtype=self.dtype, device=h.device)
        single = ctx.max_q_len == 1                # a step of single tokens: the convolution moves its state on itself
        K.causal_conv_silu(proj, self.inner, self.conv_w, self.conv_b, cache.state, self.scan_elements, ctx.q_start, ctx.seq_of_token,
                           ctx.state_slots, xbc, shift=single)
        if not single:
            K.conv_state_shift(proj, self.inner, self.channels, self.taps, cache.state, self.scan_elements, ctx.q_start, ctx.state_slots)
        y32 = torch.empty((T, self.inner), dtype=torch.float32, device=h.device)
        K.ssm_scan(xbc, proj, self.inner + self.channels, self.dt_bias, self.A_log, self.D, cache.state, ctx.q_start, ctx.state_slots, y32,
                   self.heads, self.head_dim, self.state_size, self.groups, chunks=scan_chunks(ctx))
        y = torch.empty((T, self.inner), dtype=self.dtype, device=h.device)
        K.gated_rmsnorm(y32, proj, 0, self.norm_weight, self.eps, self.norm_groups, True, y)
        return self.out(y)


@MIXERS.register("channel_ssm")
class ChannelStateSpace(Mixer):
    """Selective state-space mixer with a state row per channel (every channel and state element has its own decay).

    One product of the input gives ``[x: inner | z: inner]``.  x passes a causal convolution per channel over the last
    ``conv`` inputs (weights ``[inner, conv]``, the last column the current token's, a bias, zeros before the first token)
    and silu.  A second product of that x gives ``[dt: dt_rank | B: N | C: N]``; ``dt = softplus(W_dt dt + dt_bias)``, one
    per channel.  With ``A = -exp(A_log)`` ([inner, N]) and zeros before the first token, per channel c:

        S_t[c, :] = exp(dt_c A[c, :]) S_(t-1)[c, :] + dt_c x_c B_t,        y_t[c] = S_t[c, :] . C_t + D_c x_c.

    y is multiplied by silu(z) and mapped out.  Step sizes (a float32 product), decays, the state and the sums of the
    recurrence are float32.  A request's state slot holds S and, behind it, the last ``conv - 1`` inputs of the
    convolution.  The map of the step sizes reads the whole [dt | B | C] row with zero columns under B and C, so that it
    takes the second product's result as it stands."""

    decodes_from_device = True

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.inner = int(spec["inner"])
        self.state_size = int(spec["state_size"])
        self.dt_rank = int(spec["dt_rank"])
        self.taps = int(spec["conv"])
        n = dict(spec.get("names", {}))
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        self.low = self.dt_rank + 2 * self.state_size
        self.inp = FusedLinear(prefix, [n.get("in", "in_proj")], self.hidden, [2 * self.inner], False, dtype, suffixes=suffixes)
        self.x_proj = FusedLinear(prefix, [n.get("x", "x_proj")], self.inner, [self.low], False, dtype, suffixes=suffixes)
        self.dt_proj = FusedLinear(prefix, [n.get("dt", "dt_proj")], self.dt_rank, [self.inner], True, dtype, suffixes=suffixes)
        self.out = FusedLinear(prefix, [n.get("o", "out_proj")], self.inner, [self.hidden], False, dtype, suffixes=suffixes)
        self.names = {k: prefix + n.get(k, d) for k, d in (("conv", "conv1d.weight"), ("conv_bias", "conv1d.bias"), ("A_log", "A_log"), ("D", "D"))}
        self.conv_w = self.conv_b = self.A_log = self.D = None
        self.scan_elements = self.inner * self.state_size

    def params(self) -> List[ParamSpec]:
        nm = self.names
        return self.inp.params() + self.x_proj.params() + self.dt_proj.params() + self.out.params() + [
            ParamSpec(nm["conv"], (self.inner, self.taps), role="vector", std=0.3),
            ParamSpec(nm["conv_bias"], (self.inner,), role="vector", std=0.1),
            ParamSpec(nm["A_log"], (self.inner, self.state_size), role="vector", std=0.5),
            ParamSpec(nm["D"], (self.inner,), role="vector", init="ones_normal"),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for lin in (self.inp, self.x_proj, self.dt_proj, self.out):
            lin.bind(tensors)
        # zero columns under B and C: the product over the whole row is the product over its first dt_rank columns
        w = self.dt_proj.weight
        wide = torch.zeros((self.inner, self.low), dtype=w.dtype, device=w.device)
        wide[:, :self.dt_rank] = w
        self.dt_proj.weight, self.dt_proj.in_features = wide.contiguous(), self.low
        nm = self.names
        self.conv_w, self.conv_b = tensors.pop(nm["conv"]), tensors.pop(nm["conv_bias"])
        self.A_log, self.D = tensors.pop(nm["A_log"]).contiguous(), tensors.pop(nm["D"])

    def cache_requirement(self):
        return FixedState((self.scan_elements + (self.taps - 1) * self.inner,), torch.float32)

    def forward(self, h, ctx, cache):
        T = h.shape[0]
        proj = self.inp(h)                                     # x | z
        x = torch.empty((T, self.inner), dtype=self.dtype, device=h.device)
        single = ctx.max_q_len == 1                # a step of single tokens: the convolution moves its state on itself
        K.causal_conv_silu(proj, 0, self.conv_w, self.conv_b, cache.state, self.scan_elements, ctx.q_start, ctx.seq_of_token,
                           ctx.state_slots, x, shift=single)
        if not single:
            K.conv_state_shift(proj, 0, self.inner, self.taps, cache.state, self.scan_elements, ctx.q_start, ctx.state_slots)
        low = self.x_proj(x)                                   # dt | B | C
        dt32 = self.dt_proj(low, out_dtype=torch.float32)
        y = torch.empty((T, self.inner), dtype=self.dtype, device=h.device)
        K.channel_scan(x, 0, low, self.dt_rank, self.dt_rank + self.state_size, dt32, proj, self.inner, self.A_log, self.D, cache.state,
                       ctx.q_start, ctx.state_slots, y, chunks=scan_chunks(ctx))
        return self.out(y)
