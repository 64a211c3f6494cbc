"""The gated delta rule with a decay per head and key channel: a linear-attention mixer whose state is corrected, not
only added to.

With the mixer's input h: q = W_q h and k = W_k h (``num_kv_heads`` heads of ``head_dim``), v = W_v h (``num_heads`` heads of
``value_dim``), no biases; head a uses q/k head ``a // (num_heads / num_kv_heads)``.  Each of q, k, v passes a short causal
convolution over time per channel (weights ``[channels, taps]``, the last column the current token's, no bias, zeros
before the first token) and silu.  q and k are then made unit vectors per head, ``x / sqrt(sum(x^2) + 1e-6)``, and q is
multiplied by ``head_dim^(-1/2)``.  ``beta = sigmoid(W_b h)``, one per head.  The decays come through a low-rank map,
``g = exp(-exp(A_log_a) softplus(W_a2 (W_a1 h) + dt_bias))``, one per head and key channel.  Per head, with S of size
``head_dim x value_dim`` and zeros before the first token,

    S <- diag(g_t) S;    u = beta_t (v_t - S^T k_t);    S <- S + k_t u_t^T;    o_t = S^T q_t

in this order, so that the read-out sees the token's own write.  Each head's o is RMS-normalised over ``value_dim`` with
one weight shared by the heads, multiplied by ``sigmoid(W_g2 (W_g1 h))`` (a low-rank map again) and mapped out.

Unit norms, beta, the decays with their softplus and exponentials, the state and every sum of the recurrence and of the
norm are float32 (the decays' second product has a float32 result).  A request's state slot holds S of every head and,
behind it, the last ``taps - 1`` inputs of the convolution; both move on by whatever the step holds of the request.
The convolution's results stay float32 on their way into the recurrence.

One product serves q | k | v | b | a1 | g1; the second products of the two low-rank maps read that row's columns through
matrices with zero columns elsewhere, so nothing is copied.  What does not depend on the state (convolution, unit vectors,
decays, beta) is made once per token by one kernel, the walk over the state is a second one.  The kernels find the step's sequences and their slots on the
device, so steps of single tokens are replayed from a captured graph.  A portion runs in one piece, token after token:
the rule is not elementwise in S (the correction mixes the key channels), so chunks of it do not run side by side.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import MIXERS, FixedState, Mixer
from .linear import FusedLinear

UNIT_EPS = 1e-6          # inside the root of the unit norms of q and k: the rule's own constant


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(Mixer):
    decodes_from_device = True

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.kv_heads = int(spec.get("num_kv_heads") or self.heads)
        self.dim = int(spec["head_dim"])
        self.value_dim = int(spec.get("value_dim") or self.dim)
        self.taps = int(spec["conv"])
        self.decay_rank = int(spec["decay_rank"])
        self.gate_rank = int(spec["gate_rank"])
        self.eps = float(spec["eps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.kv_heads} key heads")
        if self.taps < 1:
            raise ValueError(f"a convolution of {self.taps} taps")
        n = dict(spec.get("names", {}))
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        qk, vv = self.kv_heads * self.dim, self.heads * self.value_dim
        self.qk, self.vv = qk, vv
        self.channels = 2 * qk + vv                     # what the convolution runs over: q | k | v
        stems = [n.get(k, k + "_proj") for k in ("q", "k", "v", "b", "a1", "g1")]
        outs = [qk, qk, vv, self.heads, self.decay_rank, self.gate_rank]
        self.proj = FusedLinear(prefix, stems, self.hidden, outs, False, dtype, suffixes=suffixes)
        self.width = -(-sum(outs) // 8) * 8             # (zero rows up to a multiple of 8: the second products then run on the tensor cores)
        self.b_col = self.channels
        self.a1_col = self.b_col + self.heads
        self.g1_col = self.a1_col + self.decay_rank
        # the second products of the two low-rank maps: over the whole row, zero columns outside their own inputs
        self.decay_out = FusedLinear(prefix, [n.get("a2", "a2_proj")], self.decay_rank, [self.heads * self.dim], False, dtype, suffixes=suffixes)
        self.gate_out = FusedLinear(prefix, [n.get("g2", "g2_proj")], self.gate_rank, [vv], False, dtype, suffixes=suffixes)
        self.out = FusedLinear(prefix, [n.get("o", "o_proj")], vv, [self.hidden], False, dtype, suffixes=suffixes)
        self.conv_names = [prefix + n.get(k, k + "_proj") + str(spec.get("conv_suffix", ".conv")) for k in ("q", "k", "v")]
        self.names = {k: prefix + n.get(k, d) for k, d in (("dt_bias", "dt_bias"), ("A_log", "A_log"), ("norm", "norm.weight"))}
        self.conv_w = self.A_log = self.norm_weight = None
        self.scan_elements = self.heads * self.dim * self.value_dim

    def params(self) -> List[ParamSpec]:
        nm = self.names
        out = self.proj.params() + self.decay_out.params() + self.gate_out.params() + self.out.params()
        out += [ParamSpec(name, (c, self.taps), role="vector", mean=1.0 / self.taps, std=0.3) for name, c in zip(self.conv_names, (self.qk, self.qk, self.vv))]
        out += [ParamSpec(nm["dt_bias"], (self.heads * self.dim,), role="vector", std=0.5),
                ParamSpec(nm["A_log"], (self.heads,), role="vector", mean=-1.0, std=0.5),
                ParamSpec(nm["norm"], (self.value_dim,), role="vector", init="ones_normal")]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for lin in (self.proj, self.decay_out, self.gate_out, self.out):
            lin.bind(tensors)
        w = self.proj.weight
        if w.shape[0] != self.width:
            self.proj.weight = torch.cat([w, torch.zeros((self.width - w.shape[0], w.shape[1]), dtype=w.dtype, device=w.device)], dim=0).contiguous()
            self.proj.out_features = self.width
        for lin, col, rank in ((self.decay_out, self.a1_col, self.decay_rank), (self.gate_out, self.g1_col, self.gate_rank)):
            w = lin.weight
            wide = torch.zeros((w.shape[0], self.width), dtype=w.dtype, device=w.device)
            wide[:, col:col + rank] = w
            lin.weight, lin.in_features = wide.contiguous(), self.width
        nm = self.names
        self.decay_out.bias = tensors.pop(nm["dt_bias"]).contiguous()            # the decays' map ends with this addition
        self.conv_w = torch.cat([tensors.pop(name) for name in self.conv_names], dim=0).contiguous()
        self.A_log = tensors.pop(nm["A_log"]).contiguous()
        self.norm_weight = tensors.pop(nm["norm"]).repeat(self.heads).contiguous()

    def cache_requirement(self):
        return FixedState((self.scan_elements + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, h, ctx, cache):
        T = h.shape[0]
        proj = self.proj(h)                                     # q | k | v | b | a1 | g1
        za = self.decay_out(proj, out_dtype=torch.float32)      # the softplus' input, bias added
        gate = self.gate_out(proj)
        # what does not depend on the state, once per token: convolution and silu, unit vectors, decays, beta
        DP = K.delta_row_elements(self.dim)
        prep_qk = torch.empty((T, self.kv_heads, 2 * DP + 4), dtype=torch.float32, device=h.device)
        prep_g = torch.empty((T, self.heads, DP + 4), dtype=torch.float32, device=h.device)
        v32 = torch.empty((T, self.vv), dtype=torch.float32, device=h.device)
        single = ctx.max_q_len == 1                 # a step of single tokens: the convolution moves its state on itself
        K.delta_prepare(proj, 0, self.b_col, self.conv_w, cache.state, self.scan_elements, ctx.q_start, ctx.seq_of_token, ctx.state_slots, za, 0,
                        self.A_log, prep_qk, prep_g, v32, self.heads, self.kv_heads, self.dim, self.value_dim, UNIT_EPS, shift=single)
        if not single and self.taps > 1:
            K.conv_state_shift(proj, 0, self.channels, self.taps, cache.state, self.scan_elements, ctx.q_start, ctx.state_slots)
        o32 = torch.empty((T, self.vv), dtype=torch.float32, device=h.device)
        K.delta_scan(prep_qk, prep_g, v32, cache.state, ctx.q_start, ctx.state_slots, o32, self.heads, self.kv_heads, self.dim, self.value_dim)
        y = torch.empty((T, self.vv), dtype=self.dtype, device=h.device)
        K.gated_rmsnorm(o32, gate, 0, self.norm_weight, self.eps, self.heads, False, y, gate_act="sigmoid")
        return self.out(y)
