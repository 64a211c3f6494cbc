"""Configuration of the Demavik decoder, read from config.json.

config.json names the design under ``architecture`` and lists the layers one by one: each entry gives its ``type``
(which mixer it has), the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for none).  Model-wide keys:
``vocab``, ``width``, ``norm.eps``, ``residual_mult`` and ``embedding`` (``scale``: a factor on the token embedding;
``bigram``: ``buckets``, ``mul_prev``, ``mul_cur`` of an embedding of token pairs that is added to it).

A sublayer reads the residual stream itself; the norm stands on its output only, and the result is added with a constant
factor: ``x += residual_mult * rms(sublayer(x)) * w``.  In the engine's terms: a block with a norm before and after
each sublayer whose first norm is none at all (kind ``identity``) and whose second carries the factor (``gain``).

Layer types:

* ``attention``: grouped-query causal softmax attention with biased projections, an RMS norm over the whole query
  projection and the whole key projection (a weight per channel), rotation of the first ``rot.dims`` elements of each
  head (base ``rot.base``, long waves slowed down by ``rot.scaling``: factor, low, high, original), scores scaled by
  ``scale``.  With ``kv_from``: j the layer has no keys and values of its own and reads the cache of layer j.
* ``gla``: linear attention with a decay per token and key channel (``tau``; the rank of the decays' map is the shape of
  its first matrix, which config.json does not repeat: ``decay_rank`` may give it, else it is read from the file).
* ``mamba1``: a selective scan with a state row per channel (``inner``, ``state``, ``dt_rank``, ``conv`` taps).

The feed-forward (``kind`` moe) is a mixture of ``router.experts`` gated units of width ``expert.ff``, ``router.top`` of
them per token, chosen by the largest router logits (with a bias); the weights are the softmax over the chosen logits.

Tensor names follow the file: ``l<i>.`` per layer, ``mix.`` / ``mlp.`` / ``norm1`` / ``norm2`` below it, weights under
the bare stem and biases under ``<stem>.b``.  Sizes and constants all come from config.json.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .filasun import _float, _int
from .gorulorn import MAX_POSITIONS, SUFFIXES, _opt_int
from .qwen2 import ConfigError
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

# the rank of the decays' map when neither config.json nor (for a folder) the file says: random-weights mode only
DEFAULT_DECAY_RANK = 16


@dataclass(frozen=True)
class DemavikConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    embedding_scale: float
    bigram: Optional[Tuple[int, int, int]]            # (buckets, mul_prev, mul_cur)
    layers: Tuple[Mapping[str, Any], ...]
    max_positions: int = MAX_POSITIONS

    ARCHITECTURE = "Demavik"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DemavikConfig":
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: missing key 'norm' (with 'eps')")
        eps = _float(norm, "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        emb = d.get("embedding") or {}
        if not isinstance(emb, Mapping):
            raise ConfigError("config.json: 'embedding' must be an object ('scale', 'bigram')")
        bigram = emb.get("bigram")
        if bigram is not None:
            if not isinstance(bigram, Mapping):
                raise ConfigError("config.json: embedding.'bigram' must be an object with 'buckets', 'mul_prev' and 'mul_cur'")
            bigram = tuple(_int(bigram, k, "embedding.bigram.") for k in ("buckets", "mul_prev", "mul_cur"))
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), eps=eps, residual_mult=_float(d, "residual_mult", "", 1.0),
                  embedding_scale=_float(emb, "scale", "embedding.", 1.0), bigram=bigram, layers=tuple(layers),
                  max_positions=_int(d, "max_positions", "") if d.get("max_positions") is not None else MAX_POSITIONS)
        cfg.to_model_spec()                       # every layer's keys are read (and refused) here, not at the first step
        return cfg

    @staticmethod
    def sizes_from_tensors(d: Mapping[str, Any], shapes: Mapping[str, tuple]) -> Dict[str, Any]:
        """config.json with the sizes that only a tensor's shape gives written into it: the rank of a ``gla`` layer's map of
        the decays is the number of rows of its first matrix (``l<i>.mix.a1``)."""
        out = dict(d)
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)):
            return out
        new = []
        for i, layer in enumerate(layers):
            shape = shapes.get(f"l{i}.mix.a1")
            if isinstance(layer, Mapping) and layer.get("type") == "gla" and isinstance(layer.get("mixer"), Mapping) and shape and len(shape) == 2:
                layer = dict(layer, mixer=dict(layer["mixer"], decay_rank=int(shape[0])))
            new.append(layer)
        out["layers"] = new
        return out

    def to_dict(self) -> Dict[str, Any]:
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))
        out = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "residual_mult": self.residual_mult, "embedding": emb, "layers": [dict(x) for x in self.layers]}
        if self.max_positions != MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------
    def _rotation(self, m: Mapping[str, Any], dim: int, where: str) -> Optional[PartSpec]:
        rot = m.get("rot")
        if rot is None:
            return None
        if not isinstance(rot, Mapping):
            raise ConfigError(f"config.json: {where}'rot' must be an object with 'dims' and 'base'")
        dims = _int(rot, "dims", where + "rot.")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most dim {dim}")
        params: Dict[str, Any] = {"theta": _float(rot, "base", where + "rot."), "rotary_dim": dims}
        sc = rot.get("scaling")
        if sc is not None:
            if not isinstance(sc, Mapping):
                raise ConfigError(f"config.json: {where}rot.'scaling' must be an object with 'factor', 'low', 'high' and 'original'")
            params["scaling"] = {k: _float(sc, k, where + "rot.scaling.") for k in ("factor", "low", "high", "original")}
            s = params["scaling"]
            if s["factor"] <= 0 or s["high"] <= s["low"] or s["original"] <= 0:
                raise ConfigError(f"config.json: {where}rot.scaling needs factor > 0, high > low and original > 0")
        return PartSpec("rope", params)

    def _attention(self, m: Mapping[str, Any], where: str) -> PartSpec:
        heads = _int(m, "heads", where)
        kv = _opt_int(m, "kv_heads", where) or heads
        if heads % kv:
            raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv} key/value heads")
        dim = _int(m, "dim", where)
        return PartSpec("attention", {
            "hidden_size": self.width, "num_heads": heads, "num_kv_heads": kv, "head_dim": dim, "value_dim": _opt_int(m, "vdim", where) or dim,
            "scale": _float(m, "scale", where, 1.0 / math.sqrt(dim)), "window": None, "qkv_bias": True, "out_bias": False,
            "position": self._rotation(m, dim, where), "qk_norm": {"q": "q.norm", "k": "k.norm", "eps": self.eps, "whole": True},
            "shared_kv": m.get("kv_from") is not None, "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "suffixes": SUFFIXES})

    def _gla(self, m: Mapping[str, Any], where: str) -> PartSpec:
        dim = _int(m, "dim", where)
        return PartSpec("gated_linear_attention", {
            "hidden_size": self.width, "num_heads": _int(m, "heads", where), "head_dim": dim, "value_dim": _opt_int(m, "vdim", where) or dim,
            "tau": _float(m, "tau", where), "decay_rank": _opt_int(m, "decay_rank", where) or DEFAULT_DECAY_RANK, "eps": self.eps,
            "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a1": "a1", "a2": "a2", "norm": "norm"}, "suffixes": SUFFIXES})

    def _mamba1(self, m: Mapping[str, Any], where: str) -> PartSpec:
        return PartSpec("channel_ssm", {
            "hidden_size": self.width, "inner": _int(m, "inner", where), "state_size": _int(m, "state", where),
            "dt_rank": _int(m, "dt_rank", where), "conv": _int(m, "conv", where),
            "names": {"in": "in", "x": "x", "dt": "dt", "o": "o", "conv": "conv", "conv_bias": "conv.b", "A_log": "A_log", "D": "D"},
            "suffixes": SUFFIXES})

    def _mixer(self, layer: Mapping[str, Any], where: str) -> PartSpec:
        kind, m = layer.get("type"), layer.get("mixer")
        if not isinstance(m, Mapping):
            raise ConfigError(f"config.json: {where}'mixer' is missing")
        if kind == "attention":
            return self._attention(m, where + "mixer.")
        if kind == "gla":
            return self._gla(m, where + "mixer.")
        if kind == "mamba1":
            return self._mamba1(m, where + "mixer.")
        raise ConfigError(f"config.json: {where}layer type {kind!r} is not supported (attention, gla, mamba1)")

    def _feed_forward(self, layer: Mapping[str, Any], where: str) -> Optional[PartSpec]:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
            raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not supported (moe)")
        router, expert = mlp.get("router"), mlp.get("expert")
        if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
            raise ConfigError(f"config.json: {where}mlp needs 'router' (experts, top) and 'expert' (ff)")
        experts, top = _int(router, "experts", where + "mlp.router."), _int(router, "top", where + "mlp.router.")
        if top > experts:
            raise ConfigError(f"config.json: {where}mlp.router.top {top} is more than the {experts} experts")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": _int(expert, "ff", where + "mlp.expert."), "experts": experts, "top": top,
            "scoring": "softmax_chosen", "router_bias": True, "renormalize": False, "weight_on": "output",
            "names": {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"}, "suffixes": SUFFIXES})

    def schedule(self) -> Tuple[ScheduleEntry, ...]:
        """The layers in order; a layer with ``kv_from`` reads the cache of that layer's entry, which must be an attention
        layer before it with keys and values of its own and the same head counts, sizes and rotation."""
        out = []
        for i, layer in enumerate(self.layers):
            m = layer.get("mixer") if isinstance(layer, Mapping) else None
            src = m.get("kv_from") if isinstance(m, Mapping) and layer.get("type") == "attention" else None
            if src is None:
                out.append(ScheduleEntry(i))
                continue
            where = f"layers[{i}].mixer."
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                raise ConfigError(f"config.json: {where}kv_from {src!r} must name a layer before this one")
            other = self.layers[src]
            om = other.get("mixer") if isinstance(other, Mapping) else None
            if other.get("type") != "attention" or not isinstance(om, Mapping) or om.get("kv_from") is not None:
                raise ConfigError(f"config.json: {where}kv_from names layer {src}, which is no attention layer with keys and values of its own")
            for key in ("heads", "kv_heads", "dim", "vdim", "rot"):
                if om.get(key) != m.get(key):
                    raise ConfigError(f"config.json: {where}'{key}' differs from layer {src}'s, whose keys and values this layer reads")
            out.append(ScheduleEntry(i, cache_from=src))
        return tuple(out)

    def to_model_spec(self) -> ModelSpec:
        def norm(tensor, gain=1.0):
            return PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": tensor, "gain": gain})

        none = PartSpec("identity", {"size": self.width})
        blocks = []
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            where = f"layers[{i}]."
            ff = self._feed_forward(layer, where)
            blocks.append(BlockSpec.of(
                "sandwich", f"l{i}.",
                prefixes={"mixer": "mix.", "feed_forward": "mlp.", "mixer_norm": "", "mixer_post_norm": "", "feed_forward_norm": "",
                          "feed_forward_post_norm": ""},
                mixer=self._mixer(layer, where), feed_forward=ff, mixer_norm=none, mixer_post_norm=norm("norm1", self.residual_mult),
                feed_forward_norm=none if ff else None, feed_forward_post_norm=norm("norm2", self.residual_mult) if ff else None))
        inputs = ()
        if self.bigram is not None:
            buckets, mul_prev, mul_cur = self.bigram
            if buckets <= 0:
                raise ConfigError(f"config.json: embedding.bigram.buckets must be positive, got {buckets}")
            inputs = ((PartSpec("pair_embedding", {"hidden_size": self.width, "buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur,
                                                   "tensor": "bigram"}), ""),)
        return ModelSpec(
            architecture=self.ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks), schedule=self.schedule(),
            final_norm=norm("norm"), tie_word_embeddings=False, max_position_embeddings=self.max_positions, embedding_name="embed",
            final_norm_prefix="final.", lm_head_name="head", embedding_scale=self.embedding_scale if self.embedding_scale != 1.0 else None,
            stream_inputs=inputs)
