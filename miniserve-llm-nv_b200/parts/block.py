"""Block arrangements.  ``pre_norm``: ``h += mixer(norm(h)); h += feed_forward(norm(h))``
(miniserve/model/qwen3.py:336-346).  ``parallel``: one norm whose output both sublayers read,
``h += mixer(norm(h)) + feed_forward(norm(h))``; a layer without a feed-forward is ``h += mixer(norm(h))``.
``sandwich``: a norm on both sides of each sublayer, ``h += post(mixer(norm(h))); h += post(feed_forward(norm(h)))``.
``scaled_pre_norm``: ``pre_norm`` where what a sublayer adds is multiplied by a constant and, channel by channel, by a vector
of the layer (a layer scale): ``h += m * s1 * mixer(norm(h)); h += m * s2 * feed_forward(norm(h))``.

The residual stream ``h`` is float32 and is updated in place.  A block receives the stream
together with a *pending* ``delta`` that has not been added yet (the previous block's
feed-forward output) and returns its own pending delta, so that every residual add is fused
into the norm that follows it.

In steps of few rows (decode steps) a norm and the add before it cost two kernels that do next
to nothing.  Where the parts on both sides offer it (``parts.base``: ``fold_output_weight``,
``fold``, ``fold_input_weight``) the block leaves them out: the product before the norm adds
into the stream itself and writes ``h * norm weight`` with the rows' sums of squares, and the
product behind the norm divides its own results by the rows' root mean square.  What is handed
on is then a :class:`~.base.FoldedInput` instead of a delta.
"""

from __future__ import annotations

from typing import Any, Optional, Union

import torch

from .. import kernels
from .base import ChannelScaled, FoldedInput, NormFold, ParamSpec, Part, PostNormed, ResidualAdd, register_block
from .context import StepContext

# what a block hands on: nothing, an output still to add (or two, whose float32 sum is to be added), or a folded input
Pending = Union[None, torch.Tensor, tuple, FoldedInput, PostNormed, ChannelScaled]


def fold_between(producer, norm, consumer, ctx: StepContext) -> Optional[tuple]:
    """(norm weight, eps) if the norm between ``producer``'s last product and ``consumer``'s first can be folded
    into the two in this step, else None (parts that do not offer it, other sizes, float32, many rows)."""
    offers = (getattr(producer, "fold_output_weight", None), getattr(norm, "fold", None),
              getattr(consumer, "fold_input_weight", None))
    if None in offers:
        return None
    out_weight, in_weight = offers[0](ctx), offers[2](ctx)
    if out_weight is None or in_weight is None:
        return None
    gated = bool(getattr(consumer, "fold_input_gated", False))
    if not kernels.fold_supported(ctx.n_tokens, ctx.dtype, out_weight, in_weight, gated):
        return None
    return norm.fold()


def adds_into_stream(producer, ctx: StepContext) -> bool:
    """Whether ``producer``'s last product can add its results into the residual stream itself in this step."""
    offer = getattr(producer, "fold_output_weight", None)
    weight = offer(ctx) if offer is not None else None
    return weight is not None and kernels.add_in_product_supported(ctx.n_tokens, ctx.dtype, weight)


@register_block("pre_norm")
class PreNormBlock:
    takes_next_block = True          # forward() has the `next_block` argument and may receive a FoldedInput as `pending`

    def __init__(self, *, mixer, feed_forward, mixer_norm, feed_forward_norm) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, pending: Pending, ctx: StepContext, cache: Any,
                next_block: Any = None) -> Pending:
        """``pending`` is the block before's output that is not added yet (None: nothing), or the mixer's input
        already prepared by the block before (its norm folded into the products around it; the residual is up
        to date then).  ``next_block``: the block that runs next, whose first norm this block's feed-forward may
        fold likewise.  Returns what the next block receives as ``pending``."""
        if isinstance(pending, FoldedInput):
            normed = pending
        else:
            normed = ctx.buffer("block.normed", tuple(residual.shape), ctx.dtype)
            self.mixer_norm.add_and_norm(residual, pending, normed)
        fold = fold_between(self.mixer, self.feed_forward_norm, self.feed_forward, ctx)
        if fold is not None:
            normed = self.mixer.forward(normed, ctx, cache, fold=NormFold(residual, *fold))
        else:
            if adds_into_stream(self.mixer, ctx):
                delta = self.mixer.forward(normed, ctx, cache, fold=ResidualAdd(residual))      # None: added already
            else:
                delta = self.mixer.forward(normed, ctx, cache)
            normed = ctx.buffer("block.normed", tuple(residual.shape), ctx.dtype)      # (the mixer has read the first)
            self.feed_forward_norm.add_and_norm(residual, delta, normed)
        if next_block is not None and getattr(next_block, "takes_next_block", False):
            fold = fold_between(self.feed_forward, getattr(next_block, "mixer_norm", None), getattr(next_block, "mixer", None), ctx)
            if fold is not None:
                return self.feed_forward.forward(normed, ctx, fold=NormFold(residual, *fold))
        if adds_into_stream(self.feed_forward, ctx):
            return self.feed_forward.forward(normed, ctx, fold=ResidualAdd(residual))
        return self.feed_forward.forward(normed, ctx)


@register_block("parallel")
class ParallelBlock:
    """``x <- x + (mixer(h) + feed_forward(h))`` with ``h = norm(x)``: one norm per layer, read by both sublayers.

    Both outputs are handed on unadded, as a pair: the norm of the block that follows (or the model's last norm)
    adds their float32 sum into the stream as it reads it, so the sum never passes through the compute type.
    """

    def __init__(self, *, mixer, feed_forward, mixer_norm, feed_forward_norm=None) -> None:
        if feed_forward_norm is not None:
            raise ValueError("a parallel block has one norm; its feed-forward reads the mixer's input")
        self.mixer, self.feed_forward, self.mixer_norm = mixer, feed_forward, mixer_norm

    def parts(self):
        return [part for part in (self.mixer_norm, self.mixer, self.feed_forward) if part is not None]

    def forward(self, residual: torch.Tensor, pending: Pending, ctx: StepContext, cache: Any) -> Pending:
        if isinstance(pending, FoldedInput):
            raise TypeError("a parallel block takes its input from its own norm")
        # (a buffer of its own: the pending outputs of the layer before live in the parts' buffers until they are added here)
        normed = ctx.buffer("parallel.normed", tuple(residual.shape), ctx.dtype)
        self.mixer_norm.add_and_norm(residual, pending, normed)
        mixed = self.mixer.forward(normed, ctx, cache)
        if self.feed_forward is None:
            return mixed
        return mixed, self.feed_forward.forward(normed, ctx)


@register_block("sandwich")
class SandwichBlock:
    """``x <- x + post_1(mixer(norm_1(x)))``, then ``x <- x + post_2(feed_forward(norm_2(x)))``: every sublayer has a
    norm before it and a norm of its own output.  A layer may have no feed-forward.  With ``residual_scale`` m what a sublayer adds is
    ``m * post(...)``; with ``identity`` parts as ``norm_1`` and ``norm_2`` the sublayers read the stream itself, which is the
    arrangement that norms a sublayer's output only: ``x <- x + m * post_1(mixer(x))``.

    A sublayer's output is handed on unadded together with its output norm (:class:`~.base.PostNormed`); the norm that
    reads the stream next (this block's second, the next block's first, or the model's last) norms the output, adds it
    to the float32 stream and norms the stream in one kernel.
    """

    def __init__(self, *, mixer, feed_forward, mixer_norm, feed_forward_norm, mixer_post_norm, feed_forward_post_norm=None,
                 residual_scale: float = 1.0) -> None:
        self.residual_scale = float(residual_scale)
        if (feed_forward is None) != (feed_forward_norm is None) or (feed_forward is None) != (feed_forward_post_norm is None):
            raise ValueError("a sandwich block has a feed-forward with both of its norms, or none of the three")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.mixer_post_norm = mixer_norm, mixer_post_norm
        self.feed_forward_norm, self.feed_forward_post_norm = feed_forward_norm, feed_forward_post_norm

    def parts(self):
        every = (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward, self.feed_forward_post_norm)
        return [part for part in every if part is not None]

    def forward(self, residual: torch.Tensor, pending: Pending, ctx: StepContext, cache: Any) -> Pending:
        if isinstance(pending, FoldedInput):
            raise TypeError("a sandwich block takes its input from its own norm")
        normed = ctx.buffer("block.normed", tuple(residual.shape), ctx.dtype)
        self.mixer_norm.add_and_norm(residual, pending, normed)
        mixed = PostNormed(self.mixer.forward(normed, ctx, cache), *self.mixer_post_norm.fold(), self.residual_scale)
        if self.feed_forward is None:
            return mixed
        normed = ctx.buffer("block.normed", tuple(residual.shape), ctx.dtype)      # (the mixer has read the first)
        self.feed_forward_norm.add_and_norm(residual, mixed, normed)
        return PostNormed(self.feed_forward.forward(normed, ctx), *self.feed_forward_post_norm.fold(), self.residual_scale)


class LayerScales(Part):
    """The vectors that multiply a layer's sublayer outputs channel by channel, kept in float32 with the design's
    constant folded in."""

    def __init__(self, names: list, size: int, constant: float) -> None:
        self.names, self.size, self.constant = list(names), size, float(constant)
        self.weights: dict = {}

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(name, (self.size,), "vector") for name in self.names]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.weights = {name: (tensors[name].float() * self.constant).contiguous() for name in self.names}


@register_block("scaled_pre_norm")
class ScaledPreNormBlock:
    """``x <- x + m * s1 * mixer(norm_1(x))``, then ``x <- x + m * s2 * feed_forward(norm_2(x))`` with a constant ``m``
    (``residual_scale``) and the layer's vectors ``s1``, ``s2`` (``mixer_scale_name``, ``feed_forward_scale_name``: full tensor
    names).  A layer may have no feed-forward.  A sublayer's output is handed on unadded with its vector
    (:class:`~.base.ChannelScaled`); the norm that reads the stream next multiplies, adds in float32 and norms in one kernel.
    """

    def __init__(self, *, mixer, feed_forward, mixer_norm, feed_forward_norm, hidden_size: int, mixer_scale_name: str,
                 feed_forward_scale_name: Optional[str] = None, residual_scale: float = 1.0) -> None:
        if (feed_forward is None) != (feed_forward_norm is None) or (feed_forward is None) != (feed_forward_scale_name is None):
            raise ValueError("a scaled pre-norm block has a feed-forward with its norm and its scale, or none of the three")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.mixer_scale_name, self.feed_forward_scale_name = mixer_scale_name, feed_forward_scale_name
        names = [mixer_scale_name] + ([] if feed_forward_scale_name is None else [feed_forward_scale_name])
        self.scales = LayerScales(names, hidden_size, residual_scale)

    def parts(self):
        every = (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward, self.scales)
        return [part for part in every if part is not None]

    def forward(self, residual: torch.Tensor, pending: Pending, ctx: StepContext, cache: Any) -> Pending:
        if isinstance(pending, FoldedInput):
            raise TypeError("a scaled pre-norm block takes its input from its own norm")
        normed = ctx.buffer("block.normed", tuple(residual.shape), ctx.dtype)
        self.mixer_norm.add_and_norm(residual, pending, normed)
        mixed = ChannelScaled(self.mixer.forward(normed, ctx, cache), self.scales.weights[self.mixer_scale_name])
        if self.feed_forward is None:
            return mixed
        normed = ctx.buffer("block.normed", tuple(residual.shape), ctx.dtype)      # (the mixer has read the first)
        self.feed_forward_norm.add_and_norm(residual, mixed, normed)
        return ChannelScaled(self.feed_forward.forward(normed, ctx), self.scales.weights[self.feed_forward_scale_name])
