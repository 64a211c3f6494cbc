"""Configuration of the Pifazen decoder, read from config.json.

config.json names the design under ``architecture`` and lists the layers one by one: each entry gives its ``type``
(which mixer it has), the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for none).  A layer with
``weights_of``: j has no tensors of its own: it runs on layer j's (mixer, feed-forward, norms and factors) with a cache
or state of its own; in the engine's terms its schedule entry names layer j's block once more.  Model-wide keys:
``vocab``, ``width``, ``norm.eps``.

A layer is pre-norm with a learned factor per channel on each sublayer's output:
``x += ls1 * mixer(norm1(x))``, then ``x += ls2 * ff(norm2(x))``.  The norms are RMS norms whose weight is stored around
zero and applied as ``1 + w``.  In the engine's terms: the arrangement with a norm before and after each sublayer, whose
second "norm" is the factor per channel (kind ``channel_scale``).  The logits are the embedding table times the model's
last norm of the stream.

Layer types:

* ``channel_delta``: the gated delta rule with a decay per head and key channel (``heads``, ``kv_heads``, ``dim``, ``vdim``,
  ``conv`` taps).  The ranks of its two low-rank maps (decays, output gate) are the shapes of their first matrices, which
  config.json does not repeat: ``decay_rank`` / ``gate_rank`` may give them, else they are read from the file.
* ``latent_attention``: causal softmax attention whose keys and values come from one cached latent per token
  (``kv_rank``), queries through a latent of their own (``q_rank``), per head ``dim`` unrotated and ``rot_dim`` rotated
  query/key elements with one rotated key part shared by the heads, a gate per output element.
* ``latent_attention_2``: the same with queries straight from the input, frequencies blended by the pair's index
  (``rot.scaling``: factor, original, fast, slow) and a gate per head.

Rotation pairs element 2i with element 2i + 1 (``rot.base``, ``rot.dims`` = ``rot_dim``).  ``scale`` is taken as given.

The feed-forward is dense (``kind`` dense: one inner product of width ``ff`` with the PolyNorm activation, biases) or a
mixture (``kind`` moe): ``router.experts`` gated units with bounded operands (``expert.ff``, ``expert.limit``; the unit's
1.702 is the design's) and ``router.identity`` identity experts behind them; softmax scores over all router outputs, a
stored correction on the choice scores, ``router.groups`` (``count``, ``keep``), ``router.top`` choices, weights
renormalised and multiplied by ``router.scale``.

Tensor names follow the file: ``l<i>.`` per layer, ``mix.`` / ``mlp.`` / ``norm1`` / ``norm2`` / ``ls1`` / ``ls2`` below it,
weights under the bare stem and biases under ``<stem>.b``.  Sizes and constants all come from config.json.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .filasun import _float, _int
from .gorulorn import MAX_POSITIONS, SUFFIXES, _opt_int
from .qwen2 import ConfigError
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

GLU_ALPHA = 1.702                 # the gated unit's sigmoid(1.702 g)
# the ranks of the low-rank maps when neither config.json nor (for a folder) the file says: random-weights mode only
DEFAULT_RANK = 16


@dataclass(frozen=True)
class PifazenConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[Mapping[str, Any], ...]
    max_positions: int = MAX_POSITIONS

    ARCHITECTURE = "Pifazen"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "PifazenConfig":
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: missing key 'norm' (with 'eps')")
        eps = _float(norm, "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), eps=eps, layers=tuple(layers),
                  max_positions=_int(d, "max_positions", "") if d.get("max_positions") is not None else MAX_POSITIONS)
        cfg.to_model_spec()                       # every layer's keys are read (and refused) here, not at the first step
        return cfg

    @staticmethod
    def sizes_from_tensors(d: Mapping[str, Any], shapes: Mapping[str, tuple]) -> Dict[str, Any]:
        """config.json with the sizes that only a tensor's shape gives written into it: the ranks of a ``channel_delta``
        layer's two low-rank maps are the rows of their first matrices (``l<i>.mix.a1``, ``l<i>.mix.g1``)."""
        out = dict(d)
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)):
            return out
        new = []
        for i, layer in enumerate(layers):
            if isinstance(layer, Mapping) and layer.get("type") == "channel_delta" and isinstance(layer.get("mixer"), Mapping):
                j, hops = i, 0
                while isinstance(layers[j], Mapping) and isinstance(layers[j].get("weights_of"), int) and not isinstance(layers[j].get("weights_of"), bool) \
                        and 0 <= layers[j]["weights_of"] < len(layers) and hops < len(layers):
                    j, hops = layers[j]["weights_of"], hops + 1
                m = dict(layer["mixer"])
                for key, stem in (("decay_rank", "a1"), ("gate_rank", "g1")):
                    shape = shapes.get(f"l{j}.mix.{stem}")
                    if shape and len(shape) == 2:
                        m[key] = int(shape[0])
                layer = dict(layer, mixer=m)
            new.append(layer)
        out["layers"] = new
        return out

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [dict(x) for x in self.layers]}
        if self.max_positions != MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------
    def _rotation(self, m: Mapping[str, Any], rot_dim: int, where: str) -> Optional[PartSpec]:
        rot = m.get("rot")
        if not rot_dim:
            return None
        if not isinstance(rot, Mapping):
            raise ConfigError(f"config.json: {where}'rot' must be an object with 'dims' and 'base'")
        dims = _int(rot, "dims", where + "rot.")
        if dims % 2 or dims != rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and equal to rot_dim {rot_dim}")
        params: Dict[str, Any] = {"theta": _float(rot, "base", where + "rot."), "rotary_dim": dims, "pairing": "interleaved"}
        sc = rot.get("scaling")
        if sc is not None:
            if not isinstance(sc, Mapping):
                raise ConfigError(f"config.json: {where}rot.'scaling' must be an object with 'factor', 'original', 'fast' and 'slow'")
            params["scaling"] = dict({k: _float(sc, k, where + "rot.scaling.") for k in ("factor", "original", "fast", "slow")}, kind="yarn")
            if min(params["scaling"][k] for k in ("factor", "original", "fast", "slow")) <= 0:
                raise ConfigError(f"config.json: {where}rot.scaling needs factor, original, fast and slow > 0")
        return PartSpec("rope", params)

    def _latent_attention(self, m: Mapping[str, Any], where: str, second: bool) -> PartSpec:
        dim, rot_dim = _int(m, "dim", where), _int(m, "rot_dim", where)
        names = {"dkv": "dkv", "uk": "uk", "uv": "uv", "o": "o", "g": "g", "dkv_norm": "dkv.norm"}
        names.update({"q": "q"} if second else {"dq": "dq", "uq": "uq", "dq_norm": "dq.norm"})
        return PartSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": _int(m, "heads", where), "head_dim": dim, "rot_dim": rot_dim,
            "value_dim": _opt_int(m, "vdim", where) or dim, "q_rank": None if second else _int(m, "q_rank", where),
            "kv_rank": _int(m, "kv_rank", where), "scale": _float(m, "scale", where), "window": None, "eps": self.eps,
            "position": self._rotation(m, rot_dim, where), "gate": "head" if second else "element", "names": names, "suffixes": SUFFIXES})

    def _channel_delta(self, m: Mapping[str, Any], where: str) -> PartSpec:
        heads = _int(m, "heads", where)
        kv = _opt_int(m, "kv_heads", where) or heads
        if heads % kv:
            raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv} key heads")
        dim = _int(m, "dim", where)
        return PartSpec("gated_delta_rule", {
            "hidden_size": self.width, "num_heads": heads, "num_kv_heads": kv, "head_dim": dim, "value_dim": _opt_int(m, "vdim", where) or dim,
            "conv": _int(m, "conv", where), "decay_rank": _opt_int(m, "decay_rank", where) or DEFAULT_RANK,
            "gate_rank": _opt_int(m, "gate_rank", where) or DEFAULT_RANK, "eps": self.eps, "conv_suffix": ".conv",
            "names": {"q": "q", "k": "k", "v": "v", "b": "b", "a1": "a1", "a2": "a2", "g1": "g1", "g2": "g2", "o": "o", "dt_bias": "dt_bias",
                      "A_log": "A_log", "norm": "norm"}, "suffixes": SUFFIXES})

    def _mixer(self, layer: Mapping[str, Any], where: str) -> PartSpec:
        kind, m = layer.get("type"), layer.get("mixer")
        if not isinstance(m, Mapping):
            raise ConfigError(f"config.json: {where}'mixer' is missing")
        if kind == "channel_delta":
            return self._channel_delta(m, where + "mixer.")
        if kind == "latent_attention":
            return self._latent_attention(m, where + "mixer.", second=False)
        if kind == "latent_attention_2":
            return self._latent_attention(m, where + "mixer.", second=True)
        raise ConfigError(f"config.json: {where}layer type {kind!r} is not supported (channel_delta, latent_attention, latent_attention_2)")

    def _feed_forward(self, layer: Mapping[str, Any], where: str) -> Optional[PartSpec]:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        kind = mlp.get("kind") if isinstance(mlp, Mapping) else mlp
        if kind == "dense":
            return PartSpec("polynorm_mlp", {"hidden_size": self.width, "intermediate_size": _int(mlp, "ff", where + "mlp."), "eps": self.eps,
                                             "names": {"up": "up", "down": "down", "act": "act"}, "suffixes": SUFFIXES})
        if kind != "moe":
            raise ConfigError(f"config.json: {where}mlp.kind {kind!r} is not supported (dense, moe)")
        router, expert = mlp.get("router"), mlp.get("expert")
        if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
            raise ConfigError(f"config.json: {where}mlp needs 'router' (experts, top, ...) and 'expert' (ff, limit)")
        rw = where + "mlp.router."
        experts, top = _int(router, "experts", rw), _int(router, "top", rw)
        identity = router.get("identity") or 0                 # none, or a count that may be zero
        if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
            raise ConfigError(f"config.json: {rw}'identity' must be a count of identity experts, got {identity!r}")
        groups = router.get("groups")
        count = keep = 1
        if groups is not None:
            if not isinstance(groups, Mapping):
                raise ConfigError(f"config.json: {rw}'groups' must be an object with 'count' and 'keep'")
            count, keep = _int(groups, "count", rw + "groups."), _int(groups, "keep", rw + "groups.")
        outputs = experts + identity
        if count < 1 or outputs % count or not 1 <= keep <= count:
            raise ConfigError(f"config.json: {rw}groups: {outputs} router outputs do not form {count} equal groups of which {keep} are kept")
        if not 1 <= top <= keep * (outputs // count):
            raise ConfigError(f"config.json: {rw}top {top} is more than the {keep * (outputs // count)} router outputs of the kept groups")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": _int(expert, "ff", where + "mlp.expert."), "experts": experts, "top": top,
            "identity": identity, "scoring": "softmax_grouped", "groups": count, "keep_groups": keep, "renormalize": True,
            "route_scale": _float(router, "scale", rw, 1.0), "weight_on": "output", "activation": "glu_clamped",
            "limit": _float(expert, "limit", where + "mlp.expert."), "alpha": GLU_ALPHA,
            "names": {"router": "router", "correction": "correction", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"},
            "suffixes": SUFFIXES})

    def _owners(self) -> Tuple[int, ...]:
        """For every layer the layer whose tensors it runs on: itself, or the ``weights_of`` it names (followed through, if that
        layer names another in turn)."""
        out = []
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            src, seen = layer.get("weights_of"), {i}
            if src is None:
                out.append(i)
                continue
            while True:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(self.layers) or src in seen:
                    raise ConfigError(f"config.json: layers[{i}].weights_of {layer.get('weights_of')!r} must lead to another layer with tensors of its own")
                other = self.layers[src]
                if not isinstance(other, Mapping):
                    raise ConfigError(f"config.json: layers[{src}] must be an object")
                if other.get("weights_of") is None:
                    break
                seen.add(src)
                src = other.get("weights_of")
            for key in ("type", "mlp"):
                if other.get(key) != layer.get(key):
                    raise ConfigError(f"config.json: layers[{i}].'{key}' differs from layer {src}'s, whose tensors this layer uses")
            mine, theirs = layer.get("mixer"), other.get("mixer")
            ranks = ("decay_rank", "gate_rank")
            if not isinstance(mine, Mapping) or not isinstance(theirs, Mapping) or \
                    {k: v for k, v in mine.items() if k not in ranks} != {k: v for k, v in theirs.items() if k not in ranks}:
                raise ConfigError(f"config.json: layers[{i}].'mixer' differs from layer {src}'s, whose tensors this layer uses")
            out.append(src)
        return tuple(out)

    def to_model_spec(self) -> ModelSpec:
        def norm(tensor):
            return PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": tensor, "offset": 1.0})

        def factor(tensor):
            return PartSpec("channel_scale", {"size": self.width, "tensor": tensor})

        owners = self._owners()
        blocks, block_of = [], {}
        for i, layer in enumerate(self.layers):
            if owners[i] != i:
                continue
            where = f"layers[{i}]."
            ff = self._feed_forward(layer, where)
            block_of[i] = len(blocks)
            blocks.append(BlockSpec.of(
                "sandwich", f"l{i}.",
                prefixes={"mixer": "mix.", "feed_forward": "mlp.", "mixer_norm": "", "mixer_post_norm": "", "feed_forward_norm": "",
                          "feed_forward_post_norm": ""},
                mixer=self._mixer(layer, where), feed_forward=ff, mixer_norm=norm("norm1"), mixer_post_norm=factor("ls1"),
                feed_forward_norm=norm("norm2") if ff else None, feed_forward_post_norm=factor("ls2") if ff else None))
        schedule = tuple(ScheduleEntry(block_of[owners[i]]) for i in range(len(self.layers)))
        return ModelSpec(
            architecture=self.ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks), schedule=schedule,
            final_norm=norm("norm"), tie_word_embeddings=True, max_position_embeddings=self.max_positions, embedding_name="embed",
            final_norm_prefix="final.", lm_head_name="head")
