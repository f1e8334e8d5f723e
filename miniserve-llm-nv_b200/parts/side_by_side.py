"""A mixer made of several mixers that read the same input (``side_by_side``): the result is the sum of the members'
outputs, each times a constant of its own.  Every member keeps the cache it needs (pages for an attention, a state
vector for a recurrence): ``cache_need()`` is the tuple of the members' needs and ``forward`` receives the tuple of
their views.  The members are :class:`~.spec.PartSpec` of the mixer family, so any registered mixers can stand beside
one another; each gets ``prefix + member prefix`` before its tensor names.
"""

from __future__ import annotations

from typing import Sequence

import torch

from .. import kernels
from .base import MIXERS, ParamSpec, Part, register_mixer
from .context import StepContext


@register_mixer("side_by_side")
class SideBySide(Part):
    def __init__(self, *, prefix: str, members: Sequence) -> None:
        """``members``: (member prefix, PartSpec, scale) triples."""
        if len(members) < 2:
            raise ValueError("side_by_side: at least two members")
        self.members = [MIXERS.build(spec, prefix=prefix + member_prefix) for member_prefix, spec, _ in members]
        self.scales = [float(scale) for _, _, scale in members]

    def param_specs(self) -> list[ParamSpec]:
        return [spec for member in self.members for spec in member.param_specs()]

    def cache_need(self) -> tuple:
        return tuple(member.cache_need() if hasattr(member, "cache_need") else None for member in self.members)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for member in self.members:
            member.load({spec.name: tensors[spec.name] for spec in member.param_specs()})

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: tuple) -> torch.Tensor:
        outputs = []
        for index, (member, view) in enumerate(zip(self.members, cache)):
            # (members of one kind keep their results in the same buffers of the step: an earlier one's is copied first)
            outputs = [o.clone() if type(m) is type(member) else o for o, m in zip(outputs, self.members)]
            outputs.append(member.forward(x, ctx, view))
        out = ctx.buffer("side_by_side.out", tuple(outputs[0].shape), x.dtype)
        kernels.scaled_sum(outputs[0], self.scales[0], outputs[1], self.scales[1], out)
        for extra, scale in zip(outputs[2:], self.scales[2:]):
            kernels.scaled_sum(out, 1.0, extra, scale, out)
        return out
