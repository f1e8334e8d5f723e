"""Embedding parts: tables whose rows are added to the token embeddings as they enter the residual stream.

``token_pair`` (a hashed bigram embedding): token t adds row ``(token[t-1] * mul_prev + token[t] * mul_cur) mod buckets`` of a
table of ``buckets + 1`` rows; a sequence's first token adds the last row.  The token before a step's first one is part of
the request's state (one int32 per request: the last token + 1, 0 at admission), so steps may cut a sequence anywhere and
a decode step that takes its token from the step before on the device needs nothing from the host.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, StateNeed, register_embedding
from .context import StateView, StepContext


@register_embedding("token_pair")
class TokenPairEmbedding(Part):
    def __init__(self, *, name: str, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int) -> None:
        if buckets < 1 or mul_prev < 0 or mul_cur < 0:
            raise ValueError(f"token_pair: {buckets} buckets and the factors {mul_prev}, {mul_cur} must be positive")
        self.name, self.hidden_size = name, hidden_size
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.buckets + 1, self.hidden_size))]

    def cache_need(self) -> StateNeed:
        return StateNeed((1,), torch.int32)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]

    def add(self, residual: torch.Tensor, ctx: StepContext, cache: StateView) -> None:
        kernels.pair_embedding(ctx.token_ids, self.table, self.buckets, self.mul_prev, self.mul_cur, cache.states,
                               ctx.state_slots, ctx.query_start, ctx.request_of_token, residual)
