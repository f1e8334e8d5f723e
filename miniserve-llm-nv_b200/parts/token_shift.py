"""A mixer around another mixer that first moves every token's input towards the input of the token before it
(``token_shift``): ``h_t <- h_t + (h_(t-1) - h_t) * shift`` channel by channel, with ``h_(t-1)`` as it was before this
replacement and zeros before a sequence's first token.  The input of a request's last token is part of its state
(:class:`~.base.StateNeed` of ``hidden_size`` numbers per run, zero at admission), so that a sequence may be cut into steps
anywhere.  ``cache_need()`` is the pair (own state, the inner mixer's need); ``forward`` receives the pair of views.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import MIXERS, ParamSpec, Part, StateNeed, register_mixer
from .context import StepContext
from .spec import PartSpec


@register_mixer("token_shift")
class TokenShift(Part):
    def __init__(self, *, prefix: str, hidden_size: int, inner: PartSpec, shift_name: str = "shift") -> None:
        self.hidden_size = hidden_size
        self.name = prefix + shift_name
        self.inner = MIXERS.build(inner, prefix=prefix)
        self.shift: Optional[torch.Tensor] = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.hidden_size,), "vector")] + self.inner.param_specs()

    def cache_need(self) -> tuple:
        return (StateNeed((self.hidden_size,), torch.float32), self.inner.cache_need() if hasattr(self.inner, "cache_need") else None)

    def cache_members(self) -> list:
        return [self, self.inner]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.shift = tensors[self.name].float().contiguous()
        self.inner.load({spec.name: tensors[spec.name] for spec in self.inner.param_specs()})

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: tuple) -> torch.Tensor:
        own, inner = cache
        shifted = ctx.buffer("token_shift.out", tuple(x.shape), x.dtype)
        kernels.token_shift(x, self.shift, own.states, 0, ctx.state_slots, ctx.query_start, ctx.request_of_token, shifted)
        return self.inner.forward(shifted, ctx, inner)
