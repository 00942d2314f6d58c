"""Additions to the token embedding.

`hashed_pair`: a second table looked up by a hash of (previous token, token),

    row = (prev * mul_prev + token * mul_cur) mod buckets,     row = buckets for a request's first token,

whose row is added to the token's embedding.  The previous token of a step's first row is the last
token of the request's previous step: the request's state slot remembers it (as token + 1; a new
request's slot is zero, which says "none"), so the look-up never leaves the device and a step that
is replayed from a graph needs no extra input.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..registry import register_part
from .base import EmbeddingExtra, Fetch, StateSpec, StepContext, TensorSpec


@register_part("embedding", "hashed_pair")
class HashedPairEmbedding(EmbeddingExtra):
    graph_safe = True

    def __init__(self, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int, name: str):
        self.hidden_size, self.buckets = int(hidden_size), int(buckets)
        self.mul_prev, self.mul_cur, self.name = int(mul_prev), int(mul_cur), name
        if self.buckets < 1 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("hashed pair embedding: buckets >= 1 and multipliers >= 0")
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.buckets + 1, self.hidden_size))]

    def load(self, fetch: Fetch) -> None:
        self.table = fetch(self.name)

    def weight_bytes(self) -> int:
        return 0            # a row a token: nothing that every step reads whole

    def state_spec(self) -> StateSpec:
        return StateSpec((1,), torch.int32)

    def add(self, h: torch.Tensor, ctx: StepContext, state: Optional[torch.Tensor]) -> None:
        assert state is not None, "the hashed pair embedding needs a state slot"
        kernels.pair_hash_embed(self.table, ctx, state, h, self.buckets, self.mul_prev, self.mul_cur)
