"""Norm parts.  ``rms``: ``weight * x * rsqrt(mean(x^2) + eps)`` with the statistics in float32
(miniserve/model/layers.py:30-34), fused with the residual add that precedes it.  ``one_plus``: the stored weight
lies around zero and stands for ``1 + weight`` (added once, in float32, when the weight is loaded).  ``identity``: no norm
at all, for blocks whose sublayers read the residual stream itself: what is pending is added and the stream is handed on in
the compute type."""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ChannelScaled, ParamSpec, Part, PostNormed, register_norm


@register_norm("rms")
class RMSNorm(Part):
    def __init__(self, *, name: str, size: int, eps: float, prefix: str = "", one_plus: bool = False) -> None:
        self.name, self.size, self.eps = prefix + name, size, float(eps)
        self.one_plus = bool(one_plus)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.size,), "vector")]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]
        if self.one_plus:
            self.weight = (self.weight.float() + 1.0).contiguous()

    def add_and_norm(self, residual: torch.Tensor, delta, out: torch.Tensor,
                     rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += delta`` (float32, in place; skipped when ``delta`` is None), ``out = norm(residual)``.
        ``delta`` may be a pair of tensors (a block whose mixer and feed-forward read the same input hands on both
        outputs): the stream then receives their float32 sum.

        With ``rows`` only those rows are normalised into ``out [len(rows), size]`` and the
        residual stays as it is.
        """
        if isinstance(delta, PostNormed):
            # the output of the sublayer before passes its own norm on the way into the stream: one kernel for both
            kernels.postnorm_add_rmsnorm(residual, delta.x, delta.weight, delta.eps, self.weight, self.eps, out, rows,
                                         post_scale=delta.scale)
            return out
        if isinstance(delta, ChannelScaled):
            # the output of the sublayer before is multiplied channel by channel (in float32) on its way into the stream
            kernels.postnorm_add_rmsnorm(residual, delta.x, delta.weight, 0.0, self.weight, self.eps, out, rows, post_norm=False)
            return out
        second = None
        if isinstance(delta, tuple):
            delta, second = delta
        kernels.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows, second)
        return out

    def fold(self) -> tuple[torch.Tensor, float]:
        """(weight, eps): all that the products around this norm need to carry it out between them."""
        return self.weight, self.eps

    def norm(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """Norm over the last dim of ``x`` (any leading shape) without a residual."""
        kernels.rmsnorm(x, self.weight, self.eps, out)
        return out


@register_norm("identity")
class IdentityNorm(Part):
    """The place of a norm in a block whose sublayers read the stream as it is (designs that norm a sublayer's output
    only): ``add_and_norm`` adds what is pending into the float32 stream and writes the stream, rounded once to the compute
    type, to ``out``.  It has no tensors."""

    def __init__(self, *, size: int, prefix: str = "") -> None:
        self.size = size

    def add_and_norm(self, residual: torch.Tensor, delta, out: torch.Tensor,
                     rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if delta is None:
            kernels.postnorm_add_rmsnorm(residual, None, None, 0.0, None, 0.0, out, rows)
        elif isinstance(delta, PostNormed):
            kernels.postnorm_add_rmsnorm(residual, delta.x, delta.weight, delta.eps, None, 0.0, out, rows, post_scale=delta.scale)
        else:
            raise TypeError("the identity norm adds nothing, or an output that passes a norm of its own")
        return out
