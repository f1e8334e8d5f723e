"""A mixer made of several mixers that read the same input (``side_by_side``): the result is the sum of the members'
outputs, each times a constant of its own.  Every member keeps the cache it needs (pages for an attention, a state
vector for a recurrence): ``cache_need()`` is the tuple of the members' needs and ``forward`` receives the tuple of
their views.  The members are :class:`~.spec.PartSpec` of the mixer family, so any registered mixers can stand beside
one another; each gets ``prefix + member prefix`` before its tensor names.  With ``output_norms`` (one tensor name per member,
after ``prefix``; two members) every member's output is first divided by its root mean square over the model width and
multiplied by that weight: the result is ``sum_i scale_i * w_i * out_i / rms(out_i)``.
"""

from __future__ import annotations

from typing import Sequence

import torch

from .. import kernels
from .base import MIXERS, ParamSpec, Part, register_mixer
from .context import StepContext


@register_mixer("side_by_side")
class SideBySide(Part):
    def __init__(self, *, prefix: str, members: Sequence, output_norms: Sequence = (), hidden_size: int = 0, eps: float = 0.0) -> None:
        """``members``: (member prefix, PartSpec, scale) triples."""
        if len(members) < 2:
            raise ValueError("side_by_side: at least two members")
        self.members = [MIXERS.build(spec, prefix=prefix + member_prefix) for member_prefix, spec, _ in members]
        self.scales = [float(scale) for _, _, scale in members]
        self.norm_names = [prefix + name for name in output_norms]
        if self.norm_names and (len(self.norm_names) != 2 or len(members) != 2 or hidden_size < 1):
            raise ValueError("side_by_side: output norms are implemented for two members, one weight of the model width each")
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.norm_weights: list = []

    def param_specs(self) -> list[ParamSpec]:
        own = [ParamSpec(name, (self.hidden_size,), "vector") for name in self.norm_names]
        return [spec for member in self.members for spec in member.param_specs()] + own

    def cache_need(self) -> tuple:
        return tuple(member.cache_need() if hasattr(member, "cache_need") else None for member in self.members)

    def cache_members(self) -> list:
        """The parts that the entries of :meth:`cache_need` belong to, in its order."""
        return list(self.members)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for member in self.members:
            member.load({spec.name: tensors[spec.name] for spec in member.param_specs()})
        self.norm_weights = [tensors[name].float().contiguous() for name in self.norm_names]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: tuple) -> torch.Tensor:
        outputs = []
        for index, (member, view) in enumerate(zip(self.members, cache)):
            # (members of one kind keep their results in the same buffers of the step: an earlier one's is copied first)
            outputs = [o.clone() if type(m) is type(member) else o for o, m in zip(outputs, self.members)]
            outputs.append(member.forward(x, ctx, view))
        out = ctx.buffer("side_by_side.out", tuple(outputs[0].shape), x.dtype)
        if self.norm_weights:
            kernels.normed_sum(outputs[0], self.norm_weights[0], self.scales[0], outputs[1], self.norm_weights[1], self.scales[1],
                               self.eps, out)
            return out
        kernels.scaled_sum(outputs[0], self.scales[0], outputs[1], self.scales[1], out)
        for extra, scale in zip(outputs[2:], self.scales[2:]):
            kernels.scaled_sum(out, 1.0, extra, scale, out)
        return out
