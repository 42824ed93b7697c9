"""What an arrangement adds to the embedded tokens before the first layer, beyond the multiplier
and the learned position table that the embedding kernel takes itself.

`pair_hash`: a second table whose row is chosen by a hash of (previous token, token):
    row = (previous * mul_prev + token * mul_cur) mod buckets,
and the table's last row (number `buckets`) for a sequence's first token.  The previous token of a
sequence is per-sequence state (`StateRequest`, one int32), so a sequence may go on in any step,
also with tokens that the host has not seen (tokens selected on the device)."""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.requests import StateRequest
from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .registry import register_embedding_addend
from .runtime import Runtime


@register_embedding_addend("pair_hash")
class PairHashEmbedding:
    """Parameters: `name` (the table's tensor name), `hidden_size`, `vocab_size`, `buckets`,
    `mul_prev`, `mul_cur`.  Interface of every embedding addend: `expected_tensors(spec)` (a class
    method), `load(weights)`, `cache_request()`, `bind_cache(view)` and `forward(batch, x)`, which
    adds to the 32-bit stream `x` [tokens, hidden] in place."""
    graph_safe = True
    state_attributes = ("last_token",)

    def __init__(self, spec: PartSpec, rt: Runtime):
        p = spec.params
        self.name = str(p["name"])
        self.hidden = int(p["hidden_size"])
        self.vocab = int(p["vocab_size"])
        self.buckets = int(p["buckets"])
        self.mul_prev = int(p["mul_prev"])
        self.mul_cur = int(p["mul_cur"])
        self.rt = rt
        self.last_token = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, TensorSpec]:
        p = spec.params
        return {str(p["name"]): TensorSpec((int(p["buckets"]) + 1, int(p["hidden_size"])))}

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        self.table = self.rt.matrix(weights[self.name])

    def cache_request(self):
        return StateRequest((1,), torch.int32)

    def bind_cache(self, view) -> None:
        self.last_token = view      # [slots, 1] int32

    def forward(self, batch, x: torch.Tensor) -> None:
        self.rt.ops.pair_embed_add(batch.tokens, batch.token_from, batch.token_src, batch.token_pos,
                                   batch.token_seq, batch.seq_slot, batch.seq_start, self.last_token, self.table,
                                   x, self.vocab, self.buckets, self.mul_prev, self.mul_cur)
