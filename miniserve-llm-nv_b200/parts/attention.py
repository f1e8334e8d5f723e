"""The attention mixer: grouped-query attention over a paged cache.

Computes what miniserve/model/qwen3.py:144-250 computes for one layer: q/k/v projections
without bias, optional RMSNorm of every q and k head over the head size before the rotation
(qwen3.py:177-178), the position encoding, the append of k and v to the cache, causal
attention by absolute position with softmax in float32 scaled by ``head_dim ** -0.5``
(qwen3.py:66, 243-248), and the output projection.  Differences in form: the three
projections run as one matrix product over a row-concatenated weight, and norm, rotation and
append are one kernel.

All sizes are arguments.  ``window`` limits a query to the last ``window`` keys; ``scale``
overrides the score scale; ``position`` is a :class:`~.spec.PartSpec` of the position family.
``score_softcap`` c turns a scaled score s into ``c * tanh(s / c)`` and ``score_bias_slopes`` (one
number per query head) adds ``slope * (key position - query position)`` to it: position
encodings that act on the scores instead of on queries and keys.  Either of them selects the
general attention kernel.

Further options, each off by default: ``value_dim`` (value heads of another size than query and key heads; the
output projection then reads ``num_heads * value_dim`` numbers), ``sink`` (the softmax's denominator gets one more
term, ``exp(0)``: a key of score 0 that has no value, so a head can attend to nothing), ``output_gate`` (head h's
output is multiplied by ``sigmoid(W_g x)_h``, one number per head, from the same input as the projections) and
``own_kv=False`` (the layer has no key and value tensors: its run reads another run's cache, ``LayerRun.cache_of``,
with its own queries) and ``values_from_keys`` (the layer has no value tensor: a token's values are its keys as
projected, before their norm and rotation).  With any of them the projections (queries, keys and values if the layer has them, gate
logits) are one product over a row-concatenated weight padded with zero rows to a multiple of eight, followed by
``kernels.qkv_prepare`` (per-head norm, rotation, append) and ``kernels.paged_attention`` with the sink and the gate
applied as it stores.

More options of the general form: ``bias`` (the q, k, v and output projections have biases, ``<name><bias_suffix>``; those of
q, k and v are added in float32 as ``kernels.qkv_prepare`` reads the heads), ``qk_norm_weight=False`` (the per-head norm of q
and k has no weight: ``x / rms(x)``; such a norm commutes with the rotation, which turns pairs of entries and leaves a head's
root mean square as it is, so it covers designs that norm after rotating), ``output_gate="entry"`` (the concatenated heads
are multiplied entry by entry by ``sigmoid(W_g x)``, a gate of ``num_heads * value_dim`` rows, before the output projection) and
``conv_taps`` (q, k and v pass a short causal convolution per channel, ``<name><conv_suffix>`` of shape ``[channels, taps]``
without bias, directly after the projection; the last ``taps - 1`` projected rows are the request's state, so
``cache_need()`` is then the pair (pages, state)).
"""

from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

from .. import kernels
from .base import POSITIONS, FoldedInput, NormFold, PagedKVNeed, ParamSpec, Part, ResidualAdd, StateNeed, register_mixer
from .context import PagedKVView, StepContext
from .spec import PartSpec


@register_mixer("attention")
class Attention(Part):
    def __init__(self, *, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qk_norm: bool, eps: float, position: PartSpec, window: Optional[int] = None,
                 scale: Optional[float] = None, score_softcap: Optional[float] = None,
                 score_bias_slopes: Optional[Sequence[float]] = None,
                 q_name: str = "q_proj.weight", k_name: str = "k_proj.weight",
                 v_name: str = "v_proj.weight", o_name: str = "o_proj.weight", q_norm_name: str = "q_norm.weight",
                 k_norm_name: str = "k_norm.weight", value_dim: Optional[int] = None, sink: bool = False,
                 output_gate: bool = False, own_kv: bool = True, gate_name: str = "g_proj.weight",
                 values_from_keys: bool = False, bias: bool = False, bias_suffix: str = ".b", qk_norm_weight: bool = True,
                 conv_taps: Optional[int] = None, conv_suffix: str = ".conv") -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        general_form = bool(sink or output_gate or not own_kv or values_from_keys or (value_dim is not None and value_dim != head_dim)
                            or bias or conv_taps or not qk_norm_weight)
        if general_form and 1 <= head_dim <= kernels.MAX_HEAD_DIM:
            pass            # (the general form's kernels take odd head sizes too; the rotation checks its own size)
        elif head_dim % 2 or not 2 <= head_dim <= kernels.MAX_HEAD_DIM:
            # what the general attention kernel and the fused append take; the tensor-core kernels take fewer
            # sizes, and kernels.attention_kernels() says which of them a given size gets
            raise ValueError(f"head size {head_dim} is not an even number in 2..{kernels.MAX_HEAD_DIM}")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.qk_norm, self.eps = bool(qk_norm), float(eps)
        self.window = window
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.score_softcap = float(score_softcap) if score_softcap else None
        if score_bias_slopes is not None and len(score_bias_slopes) != num_heads:
            raise ValueError(f"{len(score_bias_slopes)} score bias slopes for {num_heads} query heads")
        self.score_bias_slopes = None if score_bias_slopes is None else tuple(float(s) for s in score_bias_slopes)
        self._slopes_on_device: Optional[torch.Tensor] = None
        self.position = POSITIONS.build(position, head_dim=head_dim) if "head_dim" not in position.args \
            else POSITIONS.build(position)
        self.value_dim = head_dim if value_dim is None else int(value_dim)
        if not 1 <= self.value_dim <= kernels.MAX_HEAD_DIM:
            raise ValueError(f"value head size {self.value_dim} is not in 1..{kernels.MAX_HEAD_DIM}")
        if output_gate not in (False, True, "head", "entry"):
            raise ValueError(f"output_gate is False, 'head' (True) or 'entry', not {output_gate!r}")
        self.sink, self.output_gate, self.own_kv = bool(sink), bool(output_gate), bool(own_kv)
        self.gate_per_entry = output_gate == "entry"
        self.bias, self.qk_norm_weight = bool(bias), bool(qk_norm_weight)
        self.conv_taps = int(conv_taps) if conv_taps else None
        if self.conv_taps is not None and (not own_kv or values_from_keys or not 1 <= self.conv_taps <= kernels.MAX_CONV_TAPS):
            raise ValueError(f"conv_taps {conv_taps}: 1..{kernels.MAX_CONV_TAPS} taps on a layer's own queries, keys and values")
        # the general form: one product for all projections of the input, then qkv_prepare and the general call of
        # paged_attention (the fast paths below are written for plain heads of one size)
        self.values_from_keys = bool(values_from_keys)
        if self.values_from_keys and (self.value_dim != head_dim or not self.own_kv):
            raise ValueError("values_from_keys: the values are the layer's own keys, so both have the same size")
        self.general = (self.sink or self.output_gate or not self.own_kv or self.values_from_keys or self.value_dim != head_dim
                        or self.bias or self.conv_taps is not None or not self.qk_norm_weight)
        if self.general and (self.score_softcap or self.score_bias_slopes is not None):
            raise ValueError("score modifiers are not implemented together with value_dim, sink, output_gate or own_kv=False")
        self.names = dict(q=prefix + q_name, k=prefix + k_name, v=prefix + v_name, o=prefix + o_name,
                          q_norm=prefix + q_norm_name, k_norm=prefix + k_norm_name, g=prefix + gate_name)
        for key in ("q", "k", "v", "o"):
            self.names[key + "_b"] = self.names[key] + bias_suffix
            self.names[key + "_conv"] = self.names[key] + conv_suffix
        # columns of the general form's projection: queries, keys, values, gate logits, zero padding
        q_rows = num_heads * head_dim
        kv_rows = num_kv_heads * (head_dim + (0 if self.values_from_keys else self.value_dim)) if self.own_kv else 0
        self.k_col = q_rows if self.own_kv else -1
        self.v_col = q_rows + num_kv_heads * head_dim if self.own_kv else -1
        if self.values_from_keys:
            self.v_col = self.k_col            # the value columns ARE the key columns, read before norm and rotation
        self.gate_col = q_rows + kv_rows if self.output_gate else -1
        self.gate_rows = 0 if not self.output_gate else num_heads * self.value_dim if self.gate_per_entry else num_heads
        self.in_rows = (q_rows + kv_rows + self.gate_rows + 7) // 8 * 8
        self.conv_channels = q_rows + kv_rows          # (queries, keys and values are the projection's first columns)
        self.in_bias = self.o_bias = self.conv_weight = None
        self.qkv_weight: Optional[torch.Tensor] = None
        self.o_weight: Optional[torch.Tensor] = None
        self.q_norm_weight: Optional[torch.Tensor] = None
        self.k_norm_weight: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ declaration
    def param_specs(self) -> list[ParamSpec]:
        h, d, dv = self.hidden_size, self.head_dim, self.value_dim
        specs = [ParamSpec(self.names["q"], (self.num_heads * d, h))]
        if self.own_kv:
            specs.append(ParamSpec(self.names["k"], (self.num_kv_heads * d, h)))
            if not self.values_from_keys:
                specs.append(ParamSpec(self.names["v"], (self.num_kv_heads * dv, h)))
        if self.qk_norm and self.qk_norm_weight:
            specs.append(ParamSpec(self.names["q_norm"], (d,), "vector"))
            if self.own_kv:
                specs.append(ParamSpec(self.names["k_norm"], (d,), "vector"))
        if self.output_gate:
            specs.append(ParamSpec(self.names["g"], (self.gate_rows, h)))
        specs.append(ParamSpec(self.names["o"], (h, self.num_heads * dv)))
        present = ["q"] + (["k"] if self.own_kv else []) + (["v"] if self.own_kv and not self.values_from_keys else [])
        if self.bias:
            specs += [ParamSpec(self.names[key + "_b"], (self._rows_of(key),), "vector") for key in present + ["o"]]
        if self.conv_taps is not None:
            specs += [ParamSpec(self.names[key + "_conv"], (self._rows_of(key), self.conv_taps)) for key in present]
        return specs

    def _rows_of(self, key: str) -> int:
        return {"q": self.num_heads * self.head_dim, "k": self.num_kv_heads * self.head_dim,
                "v": self.num_kv_heads * self.value_dim, "o": self.hidden_size}[key]

    def cache_need(self):
        pages = PagedKVNeed(self.num_kv_heads, self.head_dim, self.window, None if self.value_dim == self.head_dim else self.value_dim)
        if self.conv_taps is None:
            return pages
        return (pages, StateNeed(((self.conv_taps - 1) * self.conv_channels,), torch.float32))

    def cache_members(self) -> list:
        return [self, self]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.o_weight = tensors[n["o"]]
        if self.general:
            pieces = [tensors[n["q"]]] + ([tensors[n["k"]]] if self.own_kv else [])
            if self.own_kv and not self.values_from_keys:
                pieces.append(tensors[n["v"]])
            if self.output_gate:
                pieces.append(tensors[n["g"]])
            padding = self.in_rows - sum(p.shape[0] for p in pieces)
            if padding:
                pieces.append(torch.zeros((padding, self.hidden_size), dtype=pieces[0].dtype, device=pieces[0].device))
            self.qkv_weight = torch.cat(pieces, dim=0).contiguous()
            if self.qk_norm and self.qk_norm_weight:
                self.q_norm_weight = tensors[n["q_norm"]].float().contiguous()
                self.k_norm_weight = tensors[n["k_norm"]].float().contiguous() if self.own_kv else None
            elif self.qk_norm:
                self.q_norm_weight = torch.ones(self.head_dim, dtype=torch.float32, device=self.o_weight.device)
                self.k_norm_weight = self.q_norm_weight if self.own_kv else None
            present = ["q"] + (["k"] if self.own_kv else []) + (["v"] if self.own_kv and not self.values_from_keys else [])
            if self.bias:
                self.in_bias = torch.zeros(self.in_rows, dtype=torch.float32, device=self.o_weight.device)
                at = 0
                for key in present:
                    self.in_bias[at:at + self._rows_of(key)] = tensors[n[key + "_b"]].float()
                    at += self._rows_of(key)
                self.o_bias = tensors[n["o_b"]].float().contiguous()
            if self.conv_taps is not None:
                self.conv_weight = torch.cat([tensors[n[key + "_conv"]].float() for key in present], dim=0).contiguous()
                if self.in_bias is not None:
                    self.in_bias = self.in_bias[:self.conv_channels].contiguous()      # (the convolution adds it to its inputs)
            return
        self.qkv_weight = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous()
        if self.qk_norm:
            self.q_norm_weight, self.k_norm_weight = tensors[n["q_norm"]], tensors[n["k_norm"]]
            if self.q_norm_weight.dtype != self.k_norm_weight.dtype:
                self.q_norm_weight = self.q_norm_weight.float()
                self.k_norm_weight = self.k_norm_weight.float()

    # ------------------------------------------------------------------ norms folded into the projections
    def fold_input_weight(self, ctx: StepContext) -> Optional[torch.Tensor]:
        return None if self.general else self.qkv_weight

    def fold_output_weight(self, ctx: StepContext) -> Optional[torch.Tensor]:
        return None if self.general else self.o_weight

    # ------------------------------------------------------------------ work
    def forward(self, x, ctx: StepContext, cache: PagedKVView, fold: Union[None, NormFold, ResidualAdd] = None):
        """``x``: the normed input, or a :class:`FoldedInput`.  With a :class:`NormFold` the output projection adds
        into the residual stream and a :class:`FoldedInput` for the part behind the following norm is returned;
        with a :class:`ResidualAdd` it adds into the stream and nothing is returned."""
        if self.general:
            return self._forward_general(x, ctx, cache)
        stats = None
        if isinstance(x, FoldedInput):
            x, stats = x.x, x.stats
        n, d = x.shape[0], self.head_dim
        n_q, n_kv = self.num_heads, self.num_kv_heads
        slots = cache.slots if cache.writable else torch.full_like(cache.slots, -1)
        fused = self.position.fused_args(ctx)
        attended = ctx.buffer("attention.attended", (n, n_q, d), x.dtype)
        in_product = fused is not None and kernels.qkv_in_product_supported(n, x.dtype, self.qkv_weight, d, n_q, n_kv, *fused)
        if not in_product:
            qkv = ctx.buffer("attention.qkv", (n, (n_q + 2 * n_kv) * d), x.dtype)
            kernels.linear(x, self.qkv_weight, qkv, row_stats=stats)
        if in_product:
            # many rows: norm, rotation and append happen as the projection's tiles are stored
            q = ctx.buffer("attention.q", (n, n_q, d), x.dtype)
            kernels.linear_pair_qkv(x, self.qkv_weight, slots, self.q_norm_weight, self.k_norm_weight, self.eps, fused[0],
                                    cache.key_pool, cache.value_pool, n_q, n_kv, q, row_stats=stats)
            self._attend(q, ctx, cache, attended)
        elif self._decode_in_the_attention_kernel(ctx, fused, x.dtype):
            # a step of single tokens: norm, rotation and append happen inside the split-key attention kernel
            kernels.decode_attention_fused(qkv, slots, self.q_norm_weight, self.k_norm_weight, self.eps, fused[0],
                                           cache.key_pool, cache.value_pool, cache.block_tables, ctx.query_start,
                                           ctx.context_lens, ctx.max_context_len, self.scale, self.window, n_q, n_kv, d,
                                           attended)
        else:
            q = ctx.buffer("attention.q", (n, n_q, d), x.dtype)
            if fused is not None:
                cos_sin, rotary_dim, interleaved = fused
                kernels.qk_norm_rope_append(qkv, slots, self.q_norm_weight, self.k_norm_weight, self.eps, cos_sin,
                                            rotary_dim, interleaved, cache.key_pool, cache.value_pool, n_q, n_kv, d, q)
            else:
                self._append_with_external_position(qkv, slots, ctx, cache, q)
            self._attend(q, ctx, cache, attended)
        if isinstance(fold, ResidualAdd):
            kernels.linear_add(attended.view(n, n_q * d), self.o_weight, fold.residual)
            return None
        out = ctx.buffer("attention.out", (n, self.hidden_size), x.dtype)
        if fold is not None:
            partials = ctx.buffer("attention.partials", kernels.residual_partials_shape(n, *self.o_weight.shape), torch.float32)
            stats = kernels.linear_residual(attended.view(n, n_q * d), self.o_weight, fold.residual, fold.weight,
                                                 fold.eps, out, partials)
            return FoldedInput(out, stats)
        kernels.linear(attended.view(n, n_q * d), self.o_weight, out)
        return out

    def _forward_general(self, x: torch.Tensor, ctx: StepContext, cache) -> torch.Tensor:
        """The form with a sink, a gate, value heads of their own size, another run's keys and values, biases or a
        convolution on the projections."""
        n, d, dv = x.shape[0], self.head_dim, self.value_dim
        n_q, n_kv = self.num_heads, self.num_kv_heads
        state = None
        if self.conv_taps is not None:
            cache, state = cache
        if cache.writable != self.own_kv:
            raise RuntimeError("a layer with keys and values of its own writes its cache; a layer without reads another run's")
        proj = ctx.buffer("attention.proj", (n, self.in_rows), x.dtype)
        kernels.linear(x, self.qkv_weight, proj)
        heads = proj
        if state is not None:
            # queries, keys and values are the first columns: the convolution keeps their places
            heads = ctx.buffer("attention.conv", (n, self.conv_channels), x.dtype)
            kernels.causal_conv(proj, 0, self.conv_weight, None, state.states, 0, ctx.state_slots, ctx.query_start,
                                ctx.max_query_len, heads, activation="none", in_bias=self.in_bias)
        cos_sin, rotary_dim, interleaved = self.position.fused_args(ctx)
        q = ctx.buffer("attention.q", (n, n_q, d), x.dtype)
        kernels.qkv_prepare(heads, 0, self.k_col, self.v_col, n_q, n_kv, d, dv, cache.slots, self.q_norm_weight,
                            self.k_norm_weight, self.eps, cos_sin, rotary_dim, cache.key_pool, cache.value_pool, q,
                            interleaved=interleaved, bias=self.in_bias if state is None else None)
        attended = ctx.buffer("attention.attended", (n, n_q, dv), x.dtype)
        per_head = self.output_gate and not self.gate_per_entry
        kernels.paged_attention(q, cache.key_pool, cache.value_pool, cache.block_tables, ctx.request_of_token,
                                ctx.positions, ctx.query_start, ctx.context_lens, ctx.max_query_len,
                                ctx.max_context_len, self.scale, self.window, attended, ctx.host_query_start or None,
                                sink=self.sink, gate=proj if per_head else None, gate_col=max(self.gate_col, 0))
        if self.gate_per_entry:
            kernels.sigmoid_gate_mul(attended.view(n, n_q * dv), proj, self.gate_col, attended.view(n, n_q * dv))
        out = ctx.buffer("attention.out", (n, self.hidden_size), x.dtype)
        kernels.linear(attended.view(n, n_q * dv), self.o_weight, out)
        if self.o_bias is not None:
            kernels.add_bias(out, self.o_bias)
        return out

    def _attend(self, q: torch.Tensor, ctx: StepContext, cache: PagedKVView, attended: torch.Tensor) -> None:
        if self.score_bias_slopes is not None and self._slopes_on_device is None:
            self._slopes_on_device = torch.tensor(self.score_bias_slopes, dtype=torch.float32, device=q.device)
        kernels.paged_attention(q, cache.key_pool, cache.value_pool, cache.block_tables, ctx.request_of_token,
                                ctx.positions, ctx.query_start, ctx.context_lens, ctx.max_query_len,
                                ctx.max_context_len, self.scale, self.window, attended,
                                ctx.host_query_start or None, self.score_softcap, self._slopes_on_device)

    def _decode_in_the_attention_kernel(self, ctx: StepContext, fused, dtype: torch.dtype) -> bool:
        """Whether this step's norm, rotation and append run inside the attention kernel
        (``kernels.decode_attention_fused``): one token per request, a position encoding in that kernel's form (none,
        or half-split rotation over the whole head), no score modifiers, sizes that the kernel takes."""
        if ctx.max_query_len != 1 or ctx.n_tokens != ctx.n_requests or fused is None:
            return False
        if not kernels.decode_attention_fused_preferred(ctx.n_requests):
            return False
        cos_sin, rotary_dim, interleaved = fused
        if cos_sin is not None and (interleaved or rotary_dim != self.head_dim):
            return False
        if self.score_softcap or self.score_bias_slopes is not None:
            return False
        return kernels.decode_attention_fused_supported(dtype, self.head_dim, self.num_heads, self.num_kv_heads)

    def _append_with_external_position(self, qkv, slots, ctx, cache, q_out) -> None:
        """Position parts without a fused form: norm, ``position.apply``, then a plain append."""
        n, d, n_q, n_kv = qkv.shape[0], self.head_dim, self.num_heads, self.num_kv_heads
        heads = qkv.view(n, n_q + 2 * n_kv, d)
        q = heads[:, :n_q].contiguous()
        k = heads[:, n_q:n_q + n_kv].contiguous()
        if self.qk_norm:
            kernels.rmsnorm(q, self.q_norm_weight, self.eps, q)
            kernels.rmsnorm(k, self.k_norm_weight, self.eps, k)
        q, k = self.position.apply(q, k, ctx)
        packed = torch.cat([q, k, heads[:, n_q + n_kv:]], dim=1).contiguous().view(n, -1)
        kernels.qk_norm_rope_append(packed, slots, None, None, self.eps, None, 0, False, cache.key_pool,
                                    cache.value_pool, n_q, n_kv, d, q_out)
