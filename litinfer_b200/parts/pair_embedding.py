"""An embedding of token pairs, added to the residual stream after the token embedding.

Token t of a sequence takes row ``(previous token * mul_prev + token * mul_cur) mod buckets`` of a table of
``buckets + 1`` rows; a sequence's first token, which has no previous one, takes the table's last row (number
``buckets``).  The previous token of a portion's first token is the last token of the portion before: it is part of the
request's state (one int32 in its state slot), read and moved on by the kernel that adds the rows, on the device, so
that steps of single tokens are replayed from a captured graph and a step that is fed by the sampler's output on the
device needs no word from the host.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import STREAM_INPUTS, FixedState, StreamInput


@STREAM_INPUTS.register("pair_embedding")
class PairEmbedding(StreamInput):
    decodes_from_device = True

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.buckets = int(spec["buckets"])
        self.mul_prev = int(spec["mul_prev"])
        self.mul_cur = int(spec["mul_cur"])
        if self.buckets <= 0:
            raise ValueError(f"an embedding of pairs needs at least one bucket, got {self.buckets}")
        self.tensor = prefix + str(spec.get("tensor", "pairs.weight"))
        self.table = None

    def params(self) -> List[ParamSpec]:
        return [ParamSpec(self.tensor, (self.buckets + 1, self.hidden), role="matrix")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.table = tensors.pop(self.tensor)

    def cache_requirement(self):
        return FixedState((1,), torch.int32)              # the request's last token

    def add_to_stream(self, x32, ctx, cache) -> None:
        K.add_pair_rows(x32, self.table, ctx.token_ids, ctx.positions, ctx.q_start, ctx.seq_of_token, ctx.state_slots, cache.state,
                        self.mul_prev, self.mul_cur)
