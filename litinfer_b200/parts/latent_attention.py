"""Attention whose keys and values are read off one small latent per token.

With the mixer's input h, H heads of ``head_dim`` query/key and ``value_dim`` value elements, a query latent of
``q_rank`` and a key/value latent of ``kv_rank`` elements:

    c_q = rmsnorm(W_dq h) * g_q            q = W_uq c_q                  (queries through their own latent)
    c   = rmsnorm(W_dkv h) * g_kv                                        (the only thing a token leaves behind)
    k_j = W_uk c_j,  v_j = W_uv c_j        per head, laid out head by head
    s_ij = scale * q_i . k_j               for j in the window of i (i itself and the ``window - 1`` tokens before it)
    p_ij = exp(s_ij) / (exp(sink_h) + sum_j' exp(s_ij'))                 (``sink``: a learned number per head; optional)
    o_i = sum_j p_ij v_j,  output W_o on the heads side by side.  No positions enter.

Options of the spec, all off by default:

* ``rot_dim`` (with ``position``, a position part that rotates): every head's query has ``rot_dim`` more elements behind its
  ``head_dim`` unrotated ones, and W_dkv h has ``rot_dim`` more rows behind the latent's, not normalised: one rotated key part
  k^r that all heads share.  Both are rotated by the position part, and
  ``s_ij = scale * (q_i . k_j + q^r_i . k^r_j)``.  c and the rotated k^r are what is cached: the cache's head is [c | k^r].
* ``q_rank`` None: queries come straight from the input, ``q = W_q h`` (tensor ``q``), no latent of their own.
* ``gate`` "element" (W_g h has heads * value_dim rows) or "head" (heads rows): the heads' outputs side by side are multiplied
  by ``sigmoid(W_g h)``, element by element or each head by its one number, before W_o.

Only c is cached.  Neither keys nor values are ever made: since q_i . (W_uk c_j) = (W_uk^T q_i) . c_j, each head's query
is carried into the latent space once (a product per head), attention runs there as attention with one shared key/value
head of ``kv_rank`` elements whose values are its keys, and W_uv maps each head's result out (a product per head again).
The paged cache holds c both as a key row and, transposed, as a value column, which is what the attention kernels read;
its head size is ``kv_rank`` rounded up to a multiple of 16, the padding being zeros (zero rows of W_dkv and of the
norm's weight), so no sum changes.  Norms, scores and the softmax are float32.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import MIXERS, POSITIONS, Mixer, PagedKV
from .linear import FusedLinear


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.qk_dim = int(spec["head_dim"])
        self.value_dim = int(spec.get("value_dim") or self.qk_dim)
        self.q_rank = int(spec["q_rank"]) if spec.get("q_rank") else 0         # 0: queries straight from the input
        self.kv_rank = int(spec["kv_rank"])
        self.rot_dim = int(spec.get("rot_dim") or 0)
        self.latent = -(-(self.kv_rank + self.rot_dim) // 16) * 16        # the cache's head size
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.eps = float(spec["eps"])
        self.gate_kind = spec.get("gate")
        if self.gate_kind not in (None, "element", "head"):
            raise ValueError(f"latent attention at {prefix!r}: gate {self.gate_kind!r} is not supported (element, head)")
        position = spec.get("position")
        if bool(self.rot_dim) != (position is not None):
            raise ValueError(f"latent attention at {prefix!r}: a rotated part (rot_dim) and a position part go together")
        self.position = POSITIONS.build(position, prefix, dtype, device, head_dim=self.rot_dim) if position is not None else None
        if self.position is not None and getattr(self.position, "rotary_dim", self.rot_dim) != self.rot_dim:
            raise ValueError(f"latent attention at {prefix!r}: the whole rotated part of {self.rot_dim} elements is rotated, not {self.position.rotary_dim}")
        n = dict(spec.get("names", {}))
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        H = self.num_heads
        self.q_width = H * (self.qk_dim + self.rot_dim)
        # one product gives the queries (or their latent), the key/value latent with the rotated key part, and the gate
        gate_out = {None: 0, "element": H * self.value_dim, "head": H}[self.gate_kind]
        stems = [n.get("dq", "q_a_proj") if self.q_rank else n.get("q", "q_proj"), n.get("dkv", "kv_a_proj")]
        outs = [self.q_rank or self.q_width, self.kv_rank + self.rot_dim]
        if gate_out:
            stems.append(n.get("g", "g_proj"))
            outs.append(gate_out)
        self.kv_col = outs[0]
        self.gate_col = outs[0] + outs[1]
        self.down = FusedLinear(prefix, stems, self.hidden, outs, False, dtype, suffixes=suffixes)
        self.up_q = (FusedLinear(prefix, [n.get("uq", "q_b_proj")], self.q_rank, [self.q_width], False, dtype, suffixes=suffixes)
                     if self.q_rank else None)
        self.out = FusedLinear(prefix, [n.get("o", "o_proj")], H * self.value_dim, [self.hidden], False, dtype, suffixes=suffixes)
        w = suffixes[0]
        self.names = {"uk": prefix + n.get("uk", "k_b_proj") + w, "uv": prefix + n.get("uv", "v_b_proj") + w,
                      "dq_norm": prefix + n.get("dq_norm", "q_a_norm"), "dkv_norm": prefix + n.get("dkv_norm", "kv_a_norm")}
        self.sink_name = prefix + n["sink"] if n.get("sink") else None
        self.dq_norm = self.dkv_norm = self.sinks = None
        self.key_map = self.value_map = None            # per head: W_uk^T and W_uv, laid out for the products in groups
        self.ctas_per_work_unit = H
        # the form without a rotated part, straight queries or a gate: the latent alone is the cache's head (the kernels below it
        # are the ones that form was built on)
        self.plain = not self.rot_dim and self.q_rank and not self.gate_kind

    def parts(self):
        return [self.position] if self.position is not None else []

    def params(self) -> List[ParamSpec]:
        H = self.num_heads
        out = self.down.params() + (self.up_q.params() if self.up_q is not None else []) + self.out.params() + [
            ParamSpec(self.names["uk"], (H * self.qk_dim, self.kv_rank), role="matrix"),
            ParamSpec(self.names["uv"], (H * self.value_dim, self.kv_rank), role="matrix"),
            ParamSpec(self.names["dkv_norm"], (self.kv_rank,), role="vector", init="ones_normal")]
        if self.q_rank:
            out.append(ParamSpec(self.names["dq_norm"], (self.q_rank,), role="vector", init="ones_normal"))
        if self.sink_name:
            out.append(ParamSpec(self.sink_name, (H,), role="vector", std=0.5))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.down.bind(tensors)
        if self.up_q is not None:
            self.up_q.bind(tensors)
        self.out.bind(tensors)
        H, R, Rp = self.num_heads, self.kv_rank, self.latent
        uk = tensors.pop(self.names["uk"]).view(H, self.qk_dim, R)
        uv = tensors.pop(self.names["uv"]).view(H, self.value_dim, R)
        # W_uk^T per head; with a rotated part behind the latent the product writes the head's first R columns only
        rows = Rp if self.plain else R
        key_map = torch.zeros((H, rows, self.qk_dim), dtype=uk.dtype, device=uk.device)
        key_map[:, :R] = uk.transpose(1, 2)
        value_map = torch.zeros((H, self.value_dim, Rp), dtype=uv.dtype, device=uv.device)
        value_map[:, :, :R] = uv
        self.key_map, self.value_map = key_map.contiguous(), value_map.contiguous()
        if self.q_rank:
            self.dq_norm = tensors.pop(self.names["dq_norm"])
        g = tensors.pop(self.names["dkv_norm"])
        if not self.plain:
            self.dkv_norm = g.contiguous()
            w = self.down.weight
            if w.shape[0] % 8:
                # zero rows up to a multiple of 8: the products that read parts of this row find its rows on 16-byte boundaries
                pad = -w.shape[0] % 8
                self.down.weight = torch.cat([w, torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0).contiguous()
                self.down.out_features = self.down.weight.shape[0]
        else:
            self.dkv_norm = torch.cat([g, torch.zeros(Rp - R, dtype=g.dtype, device=g.device)]).contiguous()
            if Rp != R:
                # zero rows of the key/value latent's map: the padded elements of c are zeros
                w = self.down.weight
                self.down.weight = torch.cat([w, torch.zeros((Rp - R, w.shape[1]), dtype=w.dtype, device=w.device)], dim=0).contiguous()
                self.down.out_features = self.down.weight.shape[0]
        if self.sink_name:
            self.sinks = tensors.pop(self.sink_name)

    def cache_requirement(self):
        return PagedKV(1, self.latent, self.window)

    def forward(self, h, ctx, cache):
        T = h.shape[0]
        H, Rp = self.num_heads, self.latent
        view = ctx.group(cache.group)
        lat = self.down(h)                                                   # [T, q or its latent | kv latent (| rotated key part) (| gate)]
        if self.q_rank:
            cq = torch.empty((T, self.q_rank), dtype=self.dtype, device=h.device)
            K.rmsnorm_cols(lat, 0, self.q_rank, self.q_rank, self.dq_norm, self.eps, cq, 0)
            q = self.up_q(cq)                                                # [T, H * (head_dim + rot_dim)]
        else:
            q = lat                                                          # the queries are the row's first columns
        # the attention kernels' row: H queries in the latent space, then the token's key and its value
        qkv = torch.empty((T, (H + 2) * Rp), dtype=self.dtype, device=h.device)
        if self.plain:
            K.rmsnorm_cols(lat, self.q_rank, Rp, self.kv_rank, self.dkv_norm, self.eps, qkv, H * Rp, (H + 1) * Rp)
            K.grouped_linear(q, self.key_map, qkv, None, self.qk_dim, Rp)
        else:
            rot = self.position.rotary(ctx) if self.position is not None else None
            # the unrotated query into the latent space: the first kv_rank columns of each head; the kernel behind it fills
            # the rest (rotated parts, the key's and the value's latent, zeros)
            K.grouped_linear(q, self.key_map, qkv, None, self.qk_dim + self.rot_dim, Rp)
            K.latent_rope_post(lat, self.kv_col, self.kv_col + self.kv_rank, q, self.qk_dim, self.dkv_norm, self.eps, ctx.positions,
                               rot.denominators if rot else None, rot.magnitude if rot else 1.0, bool(rot and rot.interleaved), qkv, H,
                               self.kv_rank, self.rot_dim, Rp)
        K.rope_kv_write(qkv, ctx.positions, None, 0, view.slot_mapping, cache.k, cache.v, H, 1, Rp, cache.writes)
        o = torch.empty((T, H * Rp), dtype=self.dtype, device=h.device)
        K.paged_attention(
            qkv, o, cache.k, cache.v, view.block_table, ctx.q_start, ctx.ctx_lens, ctx.seq_of_token, ctx.positions,
            H, 1, Rp, self.scale, self.window, ctx.max_q_len, ctx.max_ctx_len, old_lens=ctx.old_lens, singles=ctx.num_single,
            units=ctx.attn_units, unit_slots=ctx.attn_unit_slots, sinks=self.sinks)
        heads = torch.empty((T, H * self.value_dim), dtype=self.dtype, device=h.device)
        K.grouped_linear(o, self.value_map, heads, None, Rp, self.value_dim)
        if self.gate_kind:
            K.mul_sigmoid(heads, lat, self.gate_col, 1 if self.gate_kind == "element" else self.value_dim)
        return self.out(heads)
