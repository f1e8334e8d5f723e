"""Differential attention (``differential_attention``): every head has two score maps over the same values, and the second
map's output, times a number ``lambda`` of the layer, is taken off the first's.

With ``H`` query heads over ``G`` key/value heads, queries and keys of ``d`` and values of ``dv`` entries: ``W_q`` has ``H * 2 * d``
rows and ``W_k`` ``G * 2 * d``, laid out head by head as [map 1, map 2]; ``a_m = softmax(q_m k_m^T * scale) v`` for both maps,
``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff``, ``o = a_1 - lambda a_2``, each head's ``o`` divided by its root mean square
and multiplied by ``1 - diff``; the concatenated heads times ``sigmoid(W_g x)`` entry by entry (``output_gate``), then ``W_o``.
Options: biases on q, k and v (added in float32 as the heads are read), a position part, a window, and ``chunk``: a token
sees only the keys of its own chunk of that many positions, counted from position 0 of the sequence.

How it runs: at load the rows of ``W_q`` and ``W_k`` are reordered so that all first-map heads come before all second-map
heads.  The layer is then an ordinary grouped-query attention of ``2 H`` query heads over ``2 G`` key heads whose two halves
share ``G`` value heads (key head g reads value head ``g % G``: ``PagedKVNeed.value_heads``), for which the engine's paged
attention kernels are used; the cache of such a layer holds ``2 G`` key heads and ``G`` value heads.  One kernel then combines
the two halves of the output, norms, scales and gates.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from .base import POSITIONS, PagedKVNeed, ParamSpec, Part, register_mixer
from .context import PagedKVView, StepContext
from .spec import PartSpec


@register_mixer("differential_attention")
class DifferentialAttention(Part):
    def __init__(self, *, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int,
                 scale: float, diff: float, eps: float, position: PartSpec = PartSpec("none"), window: Optional[int] = None,
                 chunk: Optional[int] = None, bias: bool = False, output_gate: bool = True, q_name: str = "q", k_name: str = "k",
                 v_name: str = "v", o_name: str = "o", gate_name: str = "g", bias_suffix: str = ".b", lq1_name: str = "lq1",
                 lk1_name: str = "lk1", lq2_name: str = "lq2", lk2_name: str = "lk2") -> None:
        if min(hidden_size, num_heads, num_kv_heads, head_dim, value_dim) < 1 or num_heads % num_kv_heads:
            raise ValueError(f"differential_attention: sizes must be positive and {num_heads} heads a multiple of {num_kv_heads}")
        if max(head_dim, value_dim) > kernels.MAX_HEAD_DIM or (chunk is not None and chunk < 1):
            raise ValueError(f"differential_attention: head sizes {head_dim}/{value_dim} (at most {kernels.MAX_HEAD_DIM}), chunk {chunk}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.value_dim = head_dim, value_dim
        self.scale, self.diff, self.eps = float(scale), float(diff), float(eps)
        self.window, self.chunk, self.bias, self.output_gate = window, chunk, bool(bias), bool(output_gate)
        self.position = POSITIONS.build(position, head_dim=head_dim) if "head_dim" not in position.args else POSITIONS.build(position)
        self.names = {key: prefix + name for key, name in dict(
            q=q_name, k=k_name, v=v_name, o=o_name, g=gate_name, q_b=q_name + bias_suffix, k_b=k_name + bias_suffix,
            v_b=v_name + bias_suffix, lq1=lq1_name, lk1=lk1_name, lq2=lq2_name, lk2=lk2_name).items()}
        # columns of the projection: queries (first maps, second maps), keys likewise, values, gate logits, zero padding
        self.k_col = 2 * num_heads * head_dim
        self.v_col = self.k_col + 2 * num_kv_heads * head_dim
        self.gate_col = self.v_col + num_kv_heads * value_dim
        self.in_rows = (self.gate_col + (num_heads * value_dim if self.output_gate else 0) + 7) // 8 * 8
        self.in_weight = self.in_bias = self.o_weight = None
        self.lam = 0.0
        self.general = True          # (what the report of attention kernels asks: the general call of paged_attention)

    @property
    def attention_heads(self) -> int:
        """Query heads as the attention kernels see them: both maps of every head."""
        return 2 * self.num_heads

    def param_specs(self) -> list[ParamSpec]:
        n, h, H, G, d, dv = self.names, self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        specs = [ParamSpec(n["q"], (H * 2 * d, h)), ParamSpec(n["k"], (G * 2 * d, h)), ParamSpec(n["v"], (G * dv, h)),
                 ParamSpec(n["o"], (h, H * dv))]
        specs += [ParamSpec(n[key], (d,), "vector") for key in ("lq1", "lk1", "lq2", "lk2")]
        if self.output_gate:
            specs.append(ParamSpec(n["g"], (H * dv, h)))
        if self.bias:
            specs += [ParamSpec(n["q_b"], (H * 2 * d,), "vector"), ParamSpec(n["k_b"], (G * 2 * d,), "vector"),
                      ParamSpec(n["v_b"], (G * dv,), "vector")]
        return specs

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(2 * self.num_kv_heads, self.head_dim, self.window,
                           None if self.value_dim == self.head_dim else self.value_dim, self.chunk, self.num_kv_heads)

    @staticmethod
    def _maps_apart(rows: torch.Tensor, heads: int, d: int) -> torch.Tensor:
        """Rows laid out head by head as [map 1, map 2] become all first maps, then all second maps."""
        return rows.view(heads, 2, d, *rows.shape[1:]).transpose(0, 1).reshape(rows.shape).contiguous()

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        n, H, G, d = self.names, self.num_heads, self.num_kv_heads, self.head_dim
        pieces = [self._maps_apart(tensors[n["q"]], H, d), self._maps_apart(tensors[n["k"]], G, d), tensors[n["v"]]]
        if self.output_gate:
            pieces.append(tensors[n["g"]])
        padding = self.in_rows - sum(p.shape[0] for p in pieces)
        if padding:
            pieces.append(torch.zeros((padding, self.hidden_size), dtype=pieces[0].dtype, device=pieces[0].device))
        self.in_weight = torch.cat(pieces, dim=0).contiguous()
        if self.bias:
            self.in_bias = torch.zeros(self.in_rows, dtype=torch.float32, device=self.in_weight.device)
            self.in_bias[:self.k_col] = self._maps_apart(tensors[n["q_b"]].float(), H, d)
            self.in_bias[self.k_col:self.v_col] = self._maps_apart(tensors[n["k_b"]].float(), G, d)
            self.in_bias[self.v_col:self.gate_col] = tensors[n["v_b"]].float()
        lq1, lk1, lq2, lk2 = (tensors[n[key]].double() for key in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff
        self.o_weight = tensors[n["o"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedKVView) -> torch.Tensor:
        n, H, G, d, dv = x.shape[0], self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        proj = ctx.buffer("differential_attention.proj", (n, self.in_rows), x.dtype)
        kernels.linear(x, self.in_weight, proj)
        cos_sin, rotary_dim, interleaved = self.position.fused_args(ctx)
        q = ctx.buffer("differential_attention.q", (n, 2 * H, d), x.dtype)
        # first-map keys, then second-map keys; both halves read the same G value heads
        key_pool, value_pool = cache.key_pool, cache.value_pool
        kernels.qkv_prepare(proj, 0, self.k_col, self.v_col, 2 * H, 2 * G, d, dv, cache.slots, None, None, self.eps, cos_sin,
                            rotary_dim, key_pool, value_pool, q, interleaved=interleaved, bias=self.in_bias, value_heads=G)
        attended = ctx.buffer("differential_attention.attended", (n, 2 * H, dv), x.dtype)
        kernels.paged_attention(q, key_pool, value_pool, cache.block_tables, ctx.request_of_token, ctx.positions,
                                ctx.query_start, ctx.context_lens, ctx.max_query_len, ctx.max_context_len, self.scale,
                                self.window, attended, ctx.host_query_start or None, chunk=self.chunk)
        combined = ctx.buffer("differential_attention.combined", (n, H, dv), x.dtype)
        kernels.differential_combine(attended, self.lam, self.eps, 1.0 - self.diff, proj if self.output_gate else None,
                                     self.gate_col, combined)
        out = ctx.buffer("differential_attention.out", (n, self.hidden_size), x.dtype)
        kernels.linear(combined.view(n, H * dv), self.o_weight, out)
        return out
