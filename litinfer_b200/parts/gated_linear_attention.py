"""Gated linear attention: linear attention whose state decays by a learned factor per token and key channel.

q = h Wq^T / sqrt(dim), k = h Wk^T ([heads, dim]), v = h Wv^T ([heads, value_dim]), no activation on any of them.  The
decays come through a low-rank map: ``z = (h Wa1^T) Wa2^T + b`` ([heads, dim]) and ``a = sigmoid(z)^(1 / tau)``.  Per head

    S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S is dim x value_dim, zeros before the first token; the decay acts on
    o_t = S_t^T q_t                             the rows that belong to key channels)

Each head's o is RMS-normalised by itself with one weight of ``value_dim`` shared by the heads, the heads side by side are
multiplied by ``silu(h Wg^T)`` and mapped out.  Decays (as logarithms, ``log sigmoid(z) / tau``), the state and every sum
of the recurrence and of the norm are float32; z itself is a float32 product.  A request's state lives in its state slot
and moves on by whatever the step holds of the request.

One product serves q | k | v | g | a1.  The kernels find the step's sequences and their slots on the device, so steps of
single tokens are replayed from a captured graph; long portions run in chunks side by side (``parts.scan``).
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import MIXERS, FixedState, Mixer
from .linear import FusedLinear
from .scan import scan_chunks


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    decodes_from_device = True

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.dim = int(spec["head_dim"])
        self.value_dim = int(spec.get("value_dim") or self.dim)
        self.rank = int(spec["decay_rank"])
        self.tau = float(spec["tau"])
        self.eps = float(spec["eps"])
        if self.tau <= 0:
            raise ValueError(f"tau must be positive, got {self.tau}")
        n = dict(spec.get("names", {}))
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        qk, vv = self.heads * self.dim, self.heads * self.value_dim
        self.qk, self.vv = qk, vv
        self.proj = FusedLinear(prefix, [n.get("q", "q_proj"), n.get("k", "k_proj"), n.get("v", "v_proj"), n.get("g", "g_proj")],
                                self.hidden, [qk, qk, vv, vv], False, dtype, suffixes=suffixes)
        # the low-rank map of the decays: its first product apart (its result is the second one's input as it stands), the
        # second with a float32 result
        self.decay_in = FusedLinear(prefix, [n.get("a1", "a_proj.0")], self.hidden, [self.rank], False, dtype, suffixes=suffixes)
        self.decay_out = FusedLinear(prefix, [n.get("a2", "a_proj.1")], self.rank, [qk], True, dtype, suffixes=suffixes)
        self.out = FusedLinear(prefix, [n.get("o", "o_proj")], vv, [self.hidden], False, dtype, suffixes=suffixes)
        self.norm_name = prefix + n.get("norm", "norm.weight")
        self.norm_weight = None                 # the shared weight, once per head, side by side

    def params(self) -> List[ParamSpec]:
        return self.proj.params() + self.decay_in.params() + self.decay_out.params() + self.out.params() + [
            ParamSpec(self.norm_name, (self.value_dim,), role="vector", init="ones_normal")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for lin in (self.proj, self.decay_in, self.decay_out, self.out):
            lin.bind(tensors)
        self.norm_weight = tensors.pop(self.norm_name).repeat(self.heads).contiguous()

    def cache_requirement(self):
        return FixedState((self.heads * self.dim * self.value_dim,), torch.float32)

    def forward(self, h, ctx, cache):
        T = h.shape[0]
        proj = self.proj(h)
        za = self.decay_out(self.decay_in(h), out_dtype=torch.float32)
        o32 = torch.empty((T, self.vv), dtype=torch.float32, device=h.device)
        K.gla_scan(proj, 0, self.qk, 2 * self.qk, za, 0, self.tau, cache.state, ctx.q_start, ctx.state_slots, o32, self.heads, self.dim,
                   self.value_dim, chunks=scan_chunks(ctx))
        y = torch.empty((T, self.vv), dtype=self.dtype, device=h.device)
        K.gated_rmsnorm(o32, proj, 2 * self.qk + self.vv, self.norm_weight, self.eps, self.heads, False, y, gate_act="silu")
        return self.out(y)
