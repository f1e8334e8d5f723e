"""Interfaces of the part families and their registries.

A *part* is a piece of a layer with its sizes and constants as constructor arguments.  It
declares the tensors it needs by name (:meth:`Part.param_specs`), receives them once they are
on the device (:meth:`Part.load`) and computes on device tensors.  It never learns which model
it is in: whatever it needs arrives as an argument or through the step context.

Families and the signature of their work method:

==============  ==========================================================================
norm            ``add_and_norm(residual, delta, out, rows=None)``: add ``delta`` (or nothing)
                into the float32 residual stream in place, write the norm of the sum to ``out``
position        ``tables(ctx)``: per-step device tables for the rotation; ``fused_args()``
mixer           ``forward(x, ctx, cache) -> y``; ``cache_need()`` says what ``cache`` must be (paged keys
                and values, paged latent vectors, a fixed-size state, nothing, or a tuple of these for a
                mixer made of several: ``cache`` is then the tuple of their views)
feed_forward    ``forward(x, ctx) -> y``
block           ``forward(residual, delta, ctx, cache) -> delta``: arranges the four above
embedding       ``add(residual, ctx, cache)``: adds rows of a table of its own to the token embeddings in the
                float32 stream; ``cache_need()`` as for a mixer (a state that a sequence carries, or None)
==============  ==========================================================================

A new part is a class registered under a name with ``register_norm`` / ``register_position``
/ ``register_mixer`` / ``register_feed_forward`` / ``register_block``; an architecture then
names it in its :class:`~.spec.PartSpec`.

Optional, for speed in steps of few rows: a norm between two matrix products can be *folded* into
them (:class:`NormFold`, :class:`FoldedInput`).  A norm offers it with ``fold()``, a mixer or
feed-forward with ``fold_output_weight(ctx)`` (its last product can add into the residual stream
and prepare the next part's input) and ``fold_input_weight(ctx)`` (its first product can take such
an input); a block uses the fold only where the norm and both neighbours offer it and
``kernels.fold_supported`` agrees, and parts that offer none of this are run as before.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch


@dataclass(frozen=True)
class ParamSpec:
    """A tensor a part needs: its name in the checkpoint, its shape and how it is kept.

    ``kind``: ``"matrix"`` is kept in the compute type (bfloat16 or float32); ``"vector"``
    (norm weights and the like) keeps 32 bits if the checkpoint stores 32 bits and takes the
    compute type otherwise; ``"matrix_f32"`` (a router) is a matrix kept in float32 whatever the
    compute type; ``"table"`` is an integer table kept as int32.
    """

    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"


@dataclass(frozen=True)
class PagedKVNeed:
    """The mixer keeps keys and values per token in pages; ``window`` keys back at most (None: all).  ``value_dim``:
    the size of a value head where it differs from the size of a key head (None: the same).  ``chunk``: a token sees only
    the keys of its own chunk of that many positions, counted from position 0 (None: no chunks).  ``value_heads``: the number
    of value heads where several key heads share one (a divisor of ``num_kv_heads``; key head g reads value head
    ``g % value_heads``; None: one per key head)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None
    chunk: Optional[int] = None
    value_heads: Optional[int] = None

    @property
    def num_value_heads(self) -> int:
        return self.num_kv_heads if self.value_heads is None else self.value_heads

    @property
    def value_head_dim(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim

    @property
    def keeps_all(self) -> bool:
        """Whether every key stays visible to later tokens (no window passes it, no chunk ends)."""
        return self.window is None and self.chunk is None

    def first_needed(self, position: int) -> int:
        """The first key that a query at ``position`` or later can still see."""
        first = 0
        if self.window is not None:
            first = max(first, position - self.window + 1)
        if self.chunk is not None:
            first = max(first, position - position % self.chunk)
        return first


@dataclass(frozen=True)
class PagedLatentNeed:
    """The mixer keeps ONE vector per token in pages: a latent of ``rank`` numbers, from which the keys and values of
    all heads are computed, followed by ``rot`` numbers of a rotated key part that all heads share."""

    rank: int
    rot: int
    window: Optional[int] = None

    @property
    def keeps_all(self) -> bool:
        return self.window is None

    def first_needed(self, position: int) -> int:
        return 0 if self.window is None else max(0, position - self.window + 1)


PAGED_NEEDS = (PagedKVNeed, PagedLatentNeed)     # needs whose cache is paged: block tables, slots, pages given back


@dataclass(frozen=True)
class StateNeed:
    """The mixer keeps one tensor of fixed ``shape`` and ``dtype`` per request (zero at admission)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class NormFold:
    """Handed to a mixer or feed-forward as ``fold=``: instead of returning its output, its last product adds it
    into ``residual`` (float32, in place) and prepares the input of the part behind the norm with ``weight`` and
    ``eps`` (``kernels.linear_residual``).  The part then returns a :class:`FoldedInput`."""

    residual: torch.Tensor
    weight: torch.Tensor
    eps: float


@dataclass
class ResidualAdd:
    """Handed to a mixer or feed-forward as ``fold=`` where the norm behind it is not folded but the part's last
    product can add its results into ``residual`` (float32, in place) as it stores them
    (``kernels.add_in_product_supported``): the part returns None, and the norm that follows reads the stream
    alone instead of adding a separate output into it first."""

    residual: torch.Tensor


@dataclass
class PostNormed:
    """What a block hands on where a sublayer's output passes a norm of its own before it is added to the stream:
    ``x`` is the output as computed, ``weight`` and ``eps`` are that norm's (``weight * x / rms(x)`` is what the stream
    receives, times ``scale`` where a design damps what its sublayers add).  The norm that reads the stream next carries
    out both in one kernel (``kernels.postnorm_add_rmsnorm``)."""

    x: torch.Tensor
    weight: torch.Tensor
    eps: float
    scale: float = 1.0


@dataclass
class ChannelScaled:
    """What a block hands on where a sublayer's output is multiplied channel by channel before it is added to the stream
    (a layer scale, with any constant of the design folded into ``weight``): the stream receives ``weight * x``, formed and
    added in float32 by the norm that reads the stream next (``kernels.postnorm_add_rmsnorm`` without its division)."""

    x: torch.Tensor
    weight: torch.Tensor


@dataclass
class FoldedInput:
    """What a part receives as ``x`` where the norm before it was folded: ``x = residual * norm weight`` and the
    statistics that its first product completes the norm with (``kernels.RowStats``)."""

    x: torch.Tensor
    stats: Any


class Part:
    """Common base: tensors declared by name, handed over after loading."""

    def param_specs(self) -> list[ParamSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receives ``{name: device tensor}`` for exactly the names of :meth:`param_specs`."""


class Registry:
    def __init__(self, family: str) -> None:
        self.family = family
        self._entries: dict[str, Callable[..., Any]] = {}

    def register(self, name: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
        def decorate(factory: Callable[..., Any]) -> Callable[..., Any]:
            self._entries[name] = factory
            return factory
        return decorate

    def build(self, spec, **context) -> Any:
        try:
            factory = self._entries[spec.kind]
        except KeyError:
            raise KeyError(f"no {self.family} part named {spec.kind!r}; registered: {sorted(self._entries)}") from None
        return factory(**context, **dict(spec.args))

    def names(self) -> list[str]:
        return sorted(self._entries)


NORMS = Registry("norm")
EMBEDDINGS = Registry("embedding")
POSITIONS = Registry("position")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed_forward")
BLOCKS = Registry("block")

register_norm = NORMS.register
register_embedding = EMBEDDINGS.register
register_position = POSITIONS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register
