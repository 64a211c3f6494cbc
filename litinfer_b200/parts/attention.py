"""Grouped-query attention over a paged cache of keys and values.

Formulas (src/llaisys/models/qwen2.cpp:613-699, src/ops/paged_attention/op.cpp:194-234):
q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv; position encoding on q and k;
k (after encoding) and v go into the cache at the token's position; query
head ``i`` reads key head ``i // (heads / kv_heads)``; the query at position p
sees keys 0..p, or with a window only those with p - t < window;
scores * scale, softmax in float32, weighted sum of v; output map without
bias unless the spec says so.  Sizes, scale, window and bias flags are
parameters of the spec; the position encoding is a part of its own, named by the spec
(``position``; None: none) and asked only through :meth:`~litinfer_b200.parts.base.Position.rotary`.
``qkv_bias`` may be ``None``: the biases then follow the file, each on its own
(LitInfer's linear takes a missing bias as none, src/llaisys/ops.cc:27-29).

Further options of the spec, all off by default:

* ``softcap``: a score s becomes ``softcap * tanh(s / softcap)`` after the scale;
* ``distance_slopes`` (one number per head): ``slope_h * (i - j)`` is taken off the score of query i and key j;
* ``head_gate`` (a tensor's stem): a map from the mixer's input to one number per head; head h's output is
  multiplied by the sigmoid of its number before the output map;
* ``value_dim``: values (and the heads of the output) of another size than queries and keys.  The cache, and the
  kernels, have one head size: queries, keys and values are padded with zero rows of their matrices up to the larger
  of the two (rounded up to a multiple of 16), and the output map gets zero columns there, which changes no sum;
* ``suffixes``: what follows a stem in the names of weights and biases;
* ``conv`` (taps; one tap is a learned factor per channel): a short causal convolution over time on every channel of q, k and v, right after the projection
  (with its bias) and before anything else: ``u'_t = sum_j w[:, j] u_(t - taps + 1 + j)`` with zeros before the
  sequence's start, no bias, no activation; the weights ``[channels, taps]`` are stored under the stem of q, k and v plus
  ``conv_suffix`` (default ``.conv``).  The last ``taps - 1`` projected rows of a request are state of fixed size: the
  mixer then asks for pages and a state slot;
* ``qk_norm`` (a mapping with the tensor names ``q`` and ``k`` below the prefix, and ``eps``): an RMS norm per head on
  queries and keys, its weight of head size shared by the heads, after the convolution and before the rotation;
  With ``whole`` true in the mapping the norm is over the whole projection instead (all heads of q at once, all of k at
  once, before they are split into heads), with a weight per channel;
* ``keep_first`` (with a window): the first keys of a sequence stay visible behind the window, at their own positions;
* ``shared_kv`` true: the layer has no keys and values of its own (no such tensors): it projects queries only and reads
  the cache that another layer's entry wrote (the schedule entry names it with ``cache_from``), keys as that layer
  normalised and rotated them.  Head counts and sizes are that layer's.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import MIXERS, POSITIONS, FixedState, Mixer, PagedKV
from .linear import FusedLinear, undefer


@MIXERS.register("attention")
class PagedAttention(Mixer):
    takes_deferred = True            # the q|k|v product applies the factor
    CACHE_WRITE_APART = 64           # tokens of a step from which the kernel behind the product leaves the cache write to another

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.ctas_per_work_unit = self.num_heads           # the kernel for long portions runs one CTA per head and entry
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.qk_dim = int(spec["head_dim"])
        self.value_dim = int(spec.get("value_dim") or self.qk_dim)
        # one head size for the cache and the kernels: see the module's text
        self.head_dim = self.qk_dim if self.value_dim == self.qk_dim else -(-max(self.qk_dim, self.value_dim) // 16) * 16
        self.scale = float(spec["scale"])
        self.softcap = float(spec.get("softcap") or 0.0)
        slopes = spec.get("distance_slopes")
        if slopes is not None and len(slopes) != self.num_heads:
            raise ValueError(f"{len(slopes)} distance slopes for {self.num_heads} heads")
        self.slopes = torch.tensor([float(x) for x in slopes], dtype=torch.float32, device=self.device) if slopes is not None else None
        self.window = spec.get("window")
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        self.taps = int(spec.get("conv") or 0)                # 0: no convolution
        qk_norm = spec.get("qk_norm")
        self.qk_norm_eps = float(qk_norm["eps"]) if qk_norm else 0.0
        self.norm_whole = bool(qk_norm.get("whole", False)) if qk_norm else False
        self.shared_kv = bool(spec.get("shared_kv", False))
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} key/value heads")
        names = spec.get("names", {})
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        self.q_dim = self.num_heads * self.head_dim
        self.kv_dim = self.num_kv_heads * self.head_dim
        stems = [names.get("q", "q_proj"), names.get("k", "k_proj"), names.get("v", "v_proj")]
        self.real_outs = (self.num_heads * self.qk_dim, self.num_kv_heads * self.qk_dim, self.num_kv_heads * self.value_dim)
        self.head_shapes = ((self.num_heads, self.qk_dim), (self.num_kv_heads, self.qk_dim), (self.num_kv_heads, self.value_dim))
        if self.norm_whole and self.taps >= 1:
            raise ValueError("a norm over the whole projection together with a convolution is not supported")
        if self.shared_kv:
            if self.taps >= 1:
                raise ValueError("a layer that shares another's keys and values cannot have a convolution")
            stems, self.real_outs, self.head_shapes = stems[:1], self.real_outs[:1], self.head_shapes[:1]
        self.qkv = FusedLinear(prefix, stems, self.hidden, list(self.real_outs), spec.get("qkv_bias", False), dtype, suffixes=suffixes)
        self.out = FusedLinear(prefix, [names.get("o", "o_proj")], self.num_heads * self.value_dim, [self.hidden],
                               bool(spec.get("out_bias", False)), dtype, suffixes=suffixes)
        gate = spec.get("head_gate")
        self.gate = FusedLinear(prefix, [gate], self.hidden, [self.num_heads], False, dtype, suffixes=suffixes) if gate else None
        position = spec.get("position")
        self.position = POSITIONS.build(position, prefix, dtype, device, head_dim=self.head_dim) if position is not None else None
        if getattr(self.position, "interleaved", False) or getattr(self.position, "magnitude", 1.0) != 1.0:
            raise ValueError(f"attention at {prefix!r}: its kernels rotate halves of a head with plain cosines and sines")
        self.conv_names = [prefix + n + str(spec.get("conv_suffix", ".conv")) for n in stems] if self.taps >= 1 else []
        self.norm_names = [prefix + str(qk_norm[n]) for n in (("q",) if self.shared_kv else ("q", "k"))] if qk_norm else []
        self.conv_weight = self.q_norm = self.k_norm = None
        # what the q|k|v product's epilogues cannot do goes through a kernel of its own behind a plain product
        self.post = self.taps >= 1 or bool(qk_norm) or self.shared_kv
        # steps of single tokens read the convolution's state through the step's device tensors: they can be captured
        self.decodes_from_device = self.taps > 1

    def params(self) -> List[ParamSpec]:
        out = self.qkv.params() + self.out.params() + (self.gate.params() if self.gate is not None else [])
        out += [ParamSpec(n, (o, self.taps), role="vector", mean=1.0 / self.taps, std=0.2) for n, o in zip(self.conv_names, self.real_outs)]
        if self.norm_whole:
            out += [ParamSpec(n, (o,), role="vector", init="ones_normal") for n, o in zip(self.norm_names, self.real_outs)]
        else:
            out += [ParamSpec(n, (self.qk_dim,), role="vector", init="ones_normal") for n in self.norm_names]
        return out

    def parts(self):
        return [self.position] if self.position is not None else []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.qkv.bind(tensors)
        self.out.bind(tensors)
        if self.gate is not None:
            self.gate.bind(tensors)
        conv = [tensors.pop(n) for n in self.conv_names]
        norms = [tensors.pop(n) for n in self.norm_names]
        if self.head_dim != self.qk_dim or self.head_dim != self.value_dim:
            self._pad_heads()
            conv = [self._pad_rows(t, *sh) for t, sh in zip(conv, self.head_shapes)]
            if self.norm_whole:
                norms = [self._pad_rows(t, *sh) for t, sh in zip(norms, self.head_shapes)]
            else:
                norms = [torch.cat([t, torch.zeros(self.head_dim - self.qk_dim, dtype=t.dtype, device=t.device)]) for t in norms]
        if conv:
            self.conv_weight = torch.cat(conv, dim=0).contiguous()
        if norms:
            self.q_norm = norms[0].contiguous()
            self.k_norm = norms[1].contiguous() if len(norms) > 1 else None

    def _pad_rows(self, t, heads, d):
        """Rows of a per-channel tensor [heads * d, ...] with zero rows up to the one head size of the cache."""
        out = torch.zeros((heads, self.head_dim) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        out[:, :d] = t.view(heads, d, *t.shape[1:])
        return out.view(heads * self.head_dim, *t.shape[1:])

    def _pad_heads(self) -> None:
        """Zero rows (q, k, v, with their biases) and zero columns (output map) up to the one head size of the cache."""
        D, nh, nkv = self.head_dim, self.num_heads, self.num_kv_heads

        def rows(t, heads, d):
            if t is None:
                return None
            out = torch.zeros((heads, D) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            out[:, :d] = t.view(heads, d, *t.shape[1:])
            return out.view(heads * D, *t.shape[1:])

        cuts, shapes = tuple(self.real_outs), self.head_shapes
        w = torch.split(self.qkv.weight, cuts, dim=0)
        self.qkv.weight = torch.cat([rows(t, *sh) for t, sh in zip(w, shapes)], dim=0).contiguous()
        if self.qkv.bias is not None:
            b = torch.split(self.qkv.bias, cuts, dim=0)
            self.qkv.bias = torch.cat([rows(t, *sh) for t, sh in zip(b, shapes)], dim=0).contiguous()
        self.qkv.out_features = self.qkv.weight.shape[0]
        o = self.out.weight.view(self.hidden, nh, self.value_dim)
        padded = torch.zeros((self.hidden, nh, D), dtype=o.dtype, device=o.device)
        padded[:, :, :self.value_dim] = o
        self.out.weight = padded.view(self.hidden, nh * D).contiguous()
        self.out.in_features = nh * D

    def cache_requirement(self):
        if self.shared_kv:
            return None                        # the schedule entry names the entry whose cache this layer reads
        paged = PagedKV(self.num_kv_heads, self.head_dim, self.window, self.keep_first)
        if self.taps > 1:
            # behind the pages: the last taps - 1 rows of the q|k|v projection, which the convolution of the next step reads
            return (paged, FixedState(((self.taps - 1) * self.qkv_width,), torch.float32))
        return paged

    @property
    def qkv_width(self) -> int:
        return (self.num_heads + 2 * self.num_kv_heads) * self.head_dim

    def fused_decode(self):
        rope = self.position.fused_decode() if self.position is not None else None
        if type(self) is not PagedAttention or rope is None or rope["rotary_dim"] != self.head_dim or self.out.bias is not None:
            return None
        if self.softcap or self.slopes is not None or self.gate is not None or self.value_dim != self.qk_dim or self.post or self.keep_first or self.shared_kv:
            return None
        return {"w_qkv": self.qkv.weight, "b_qkv": self.qkv.bias, "w_o": self.out.weight, "hidden": self.hidden, "heads": self.num_heads,
                "kv_heads": self.num_kv_heads, "head_dim": self.head_dim, "scale": self.scale, "window": self.window,
                "rope_denominators": rope["denominators"]}

    def forward(self, h, ctx, cache):
        return self.out(self._attend(h, ctx, cache))

    def forward_into(self, h, ctx, cache, tail):
        return tail.apply_linear(self.out, self._attend(h, ctx, cache))

    def _attend(self, h, ctx, cache):
        """Everything before the output projection: [tokens, heads * head_dim]."""
        state = None
        if self.taps > 1:
            cache, state = cache.parts                                 # pages, and the convolution's rows behind them
        view = ctx.group(cache.group)
        gate = self.gate(h) if self.gate is not None else None        # (a deferred activation: the product applies its factor)
        rot = self.position.rotary(ctx) if self.position is not None else None
        if self.shared_kv and (cache is None or cache.kind != "paged" or cache.writes):
            raise ValueError(f"attention at {self.prefix!r} shares another layer's keys and values: its schedule entry must name that layer's entry (cache_from)")
        if self.post and (self.norm_whole or self.shared_kv):
            # projection; the factors of the norms over the whole of q and of k; then norm, rotation and the cache write as one
            # kernel.  A layer without keys and values of its own projects queries only, into rows that attention reads as q|k|v.
            proj = self.qkv(h)
            T = proj.shape[0]
            nkv = 0 if self.shared_kv else self.num_kv_heads
            qkv = proj if not self.shared_kv else torch.empty((T, self.qkv_width), dtype=self.dtype, device=proj.device)
            rinv = None
            if self.norm_whole:
                rinv = torch.empty((T, 2), dtype=torch.float32, device=proj.device)
                ranges = [(0, self.q_dim, self.num_heads * self.qk_dim)]
                if not self.shared_kv:
                    ranges.append((self.q_dim, self.kv_dim, self.num_kv_heads * self.qk_dim))
                K.row_rinv(proj, ranges, self.qk_norm_eps, rinv)
            long_step = T >= self.CACHE_WRITE_APART and not self.shared_kv
            K.conv_norm_rope_kv(proj, qkv, self.conv_weight, None, 0, ctx.q_start, ctx.seq_of_token, ctx.state_slots, self.q_norm, self.k_norm,
                                self.qk_norm_eps, self.qk_dim, ctx.positions, rot.denominators if rot else None, rot.rotary_dim if rot else 0,
                                view.slot_mapping, cache.k, cache.v, self.num_heads, nkv, self.head_dim, cache.writes and not self.shared_kv,
                                to_cache=not long_step, row_rinv=rinv)
            if long_step and cache.writes:
                K.rope_kv_write(qkv, ctx.positions, None, 0, view.slot_mapping, cache.k, cache.v, self.num_heads, self.num_kv_heads, self.head_dim, True)
        elif self.post:
            # projection; then convolution, norm per head, rotation and the cache write as one kernel; then the state moves on
            proj = self.qkv(h)
            qkv = torch.empty_like(proj)
            # a step of single tokens: the convolution moves its state on itself
            single = ctx.max_q_len == 1 and state is not None and state.writes and cache.writes
            # a long step: keys and values go into the cache through the kernel that writes whole pieces of pages (the
            # transposed values one element at a time are slow)
            long_step = h.shape[0] >= self.CACHE_WRITE_APART
            K.conv_norm_rope_kv(proj, qkv, self.conv_weight, state.state if state is not None else None, 0, ctx.q_start, ctx.seq_of_token,
                                ctx.state_slots, self.q_norm, self.k_norm, self.qk_norm_eps, self.qk_dim, ctx.positions,
                                rot.denominators if rot else None, rot.rotary_dim if rot else 0, view.slot_mapping, cache.k, cache.v,
                                self.num_heads, self.num_kv_heads, self.head_dim, cache.writes, shift=single, to_cache=not long_step)
            if long_step and cache.writes:
                K.rope_kv_write(qkv, ctx.positions, None, 0, view.slot_mapping, cache.k, cache.v, self.num_heads, self.num_kv_heads, self.head_dim, True)
            if state is not None and state.writes and not single:
                K.conv_state_shift(proj, 0, self.qkv_width, self.taps, state.state, 0, ctx.q_start, ctx.state_slots)
        else:
            h, row_scale = undefer(h, self.qkv.weight)
            qkv = torch.empty((h.shape[0], self.qkv.out_features), dtype=self.dtype, device=h.device)
            # projection, position encoding of q and k, k and v into the cache: one call (and for few tokens one kernel)
            K.linear_rope_kv(
                h, self.qkv.weight, self.qkv.bias, qkv, ctx.positions, rot.denominators if rot else None, rot.rotary_dim if rot else 0,
                view.slot_mapping, cache.k, cache.v, self.num_heads, self.num_kv_heads, self.head_dim, cache.writes, row_scale=row_scale,
                cos_sin=rot.table if rot else None)
        o = torch.empty((h.shape[0], self.q_dim), dtype=self.dtype, device=h.device)
        K.paged_attention(
            qkv, o, cache.k, cache.v, view.block_table, ctx.q_start, ctx.ctx_lens, ctx.seq_of_token, ctx.positions,
            self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.window,
            ctx.max_q_len, ctx.max_ctx_len, old_lens=ctx.old_lens, singles=ctx.num_single,
            units=ctx.attn_units, unit_slots=ctx.attn_unit_slots, softcap=self.softcap, slopes=self.slopes, gate=gate, keep_first=self.keep_first)
        return o
