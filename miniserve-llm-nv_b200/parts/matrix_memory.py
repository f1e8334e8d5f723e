"""Mixers that carry a matrix per head from token to token.

``matrix_memory`` (the mLSTM of the xLSTM family): with ``h`` the input, ``H`` heads, queries and keys of ``d`` and values
of ``dv`` entries,

* ``q = W_q h * d^(-1/2)``, ``k = W_k h``, ``v = W_v h``; per head a log input gate ``i = c tanh((W_i h + b_i) / c)`` and a log
  forget gate ``f = logsigmoid(c tanh((W_f h + b_f) / c))`` (``c``: ``gate_cap``);
* with a running maximum ``m`` that starts at 0: ``m_t = max(f_t + m_(t-1), i_t)``,
  ``S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T``, ``n_t`` likewise with ``k_t`` alone, and
  ``o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)``;
* every head's ``o`` is divided by its root mean square, the heads are concatenated and multiplied by a weight and by
  ``sigmoid(W_g h)``; ``W_o`` maps the result back.

``delta_rule`` (the gated delta rule): ``H`` value heads over ``G`` query/key heads (head ``j`` reads query/key head
``j // (H / G)``),

* ``q``, ``k``, ``v`` = SiLU of a short causal convolution per channel of ``W_q h``, ``W_k h``, ``W_v h``; ``q`` and ``k`` are made
  unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``) and ``q`` is multiplied by ``d^(-1/2)``;
* ``beta = sigmoid(W_b h)`` and a decay ``g = exp(-exp(A_log) softplus(W_a h + dt_bias))`` per head;
* ``S <- g S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q`` (the read-out sees the token's own write);
* every head's ``o`` is divided by its root mean square, multiplied by a weight over ``dv`` that the heads share and by
  ``silu(W_g h)``; ``W_o`` maps the result back.

``delta_rule`` options: ``decay_per="channel"`` gives every head one decay per KEY channel, acting on the rows of ``S``: ``g =
exp(-exp(A_log_h) softplus(a + dt_bias))`` with ``a`` and ``dt_bias`` of ``H * d`` entries; ``decay_rank`` / ``gate_rank`` r make
the decay's and the output gate's projections products of two matrices through r numbers (``W_2 (W_1 h)``, tensors
``<name>1`` and ``<name>2``); ``gate_activation`` is ``silu`` or ``sigmoid``.

``linear_attention`` (lightning attention): ``q``, ``k``, ``v`` = SiLU of the projections, per head ``S_t = decay_h S_(t-1) + k_t
v_t^T`` with a constant of the head, ``o_t = S_t^T q_t``; the concatenated heads are divided by their root mean square TOGETHER,
multiplied by a weight and by ``sigmoid(W_g h)``; ``W_o`` maps the result back.

What a request carries from token to token is one float32 vector per layer (:class:`~.base.StateNeed`, zero at
admission): for ``matrix_memory`` the heads' matrices with ``n`` as one more column, then the heads' maxima; for
``delta_rule`` the convolution's last ``taps - 1`` inputs, then the heads' matrices.  Gates, decays, step sizes, unit
norms, the recurrence and the output norm are float32 whatever the compute type (the gates' logits come from a float32
product of their own); the wide projections are in the compute type.  Prompt portions, single tokens and mixed batches
run the same kernels, which walk each request's tokens in order from the state its slot holds
(``kernels.matrix_scan``).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, StateNeed, register_mixer
from .context import StateView, StepContext


def _pad_rows(pieces: list, width: int) -> torch.Tensor:
    """The pieces stacked row-wise, with zero rows up to a multiple of eight."""
    rows = sum(p.shape[0] for p in pieces)
    padding = (rows + 7) // 8 * 8 - rows
    if padding:
        pieces = pieces + [torch.zeros((padding, width), dtype=pieces[0].dtype, device=pieces[0].device)]
    return torch.cat(pieces, dim=0).contiguous()


@register_mixer("matrix_memory")
class MatrixMemory(Part):
    def __init__(self, *, prefix: str, hidden_size: int, heads: int, head_dim: int, value_dim: int, gate_cap: float, eps: float,
                 q_name: str = "q", k_name: str = "k", v_name: str = "v", g_name: str = "g", o_name: str = "o",
                 norm_name: str = "norm", i_name: str = "i", i_bias_name: str = "i.b", f_name: str = "f",
                 f_bias_name: str = "f.b") -> None:
        if min(hidden_size, heads, head_dim, value_dim) < 1 or not gate_cap > 0:
            raise ValueError("matrix_memory: every size and the gates' cap must be positive")
        if head_dim > kernels.MAX_MATRIX_SCAN_DIM:
            raise ValueError(f"matrix_memory: keys of {head_dim} entries exceed {kernels.MAX_MATRIX_SCAN_DIM}")
        self.hidden_size, self.heads, self.head_dim, self.value_dim = hidden_size, heads, head_dim, value_dim
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        self.q_col, self.k_col = 0, heads * head_dim
        self.v_col = 2 * heads * head_dim
        self.g_col = self.v_col + heads * value_dim
        self.matrix_state = heads * (value_dim + 1) * head_dim      # per head: value_dim columns of S and the column n
        self.names = {key: prefix + name for key, name in dict(
            q=q_name, k=k_name, v=v_name, g=g_name, o=o_name, norm=norm_name, i=i_name, i_b=i_bias_name, f=f_name,
            f_b=f_bias_name).items()}
        self.in_weight: Optional[torch.Tensor] = None
        self.gate_weight = self.gate_bias = self.norm_weight = self.o_weight = None

    def param_specs(self) -> list[ParamSpec]:
        n, h, H, d, dv = self.names, self.hidden_size, self.heads, self.head_dim, self.value_dim
        return [ParamSpec(n["q"], (H * d, h)), ParamSpec(n["k"], (H * d, h)), ParamSpec(n["v"], (H * dv, h)),
                ParamSpec(n["g"], (H * dv, h)), ParamSpec(n["o"], (h, H * dv)), ParamSpec(n["norm"], (H * dv,), "vector"),
                ParamSpec(n["i"], (H, h), "matrix_f32"), ParamSpec(n["i_b"], (H,), "vector"),
                ParamSpec(n["f"], (H, h), "matrix_f32"), ParamSpec(n["f_b"], (H,), "vector")]

    def cache_need(self) -> StateNeed:
        return StateNeed((self.matrix_state + self.heads,), torch.float32)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.in_weight = _pad_rows([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]]], self.hidden_size)
        self.gate_weight = torch.cat([tensors[n["i"]].float(), tensors[n["f"]].float()], dim=0).contiguous()
        self.gate_bias = torch.cat([tensors[n["i_b"]].float(), tensors[n["f_b"]].float()]).contiguous()
        self.norm_weight = tensors[n["norm"]].float().contiguous()
        self.o_weight = tensors[n["o"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateView) -> torch.Tensor:
        n, H, d, dv = x.shape[0], self.heads, self.head_dim, self.value_dim
        proj = ctx.buffer("matrix_memory.proj", (n, self.in_weight.shape[0]), x.dtype)
        kernels.linear(x, self.in_weight, proj)
        logits = ctx.buffer("matrix_memory.logits", (n, 2 * H), torch.float32)
        kernels.small_linear_f32(x, self.gate_weight, self.gate_bias, logits)
        gates = ctx.buffer("matrix_memory.gates", (n, H, 3), torch.float32)
        kernels.exponential_gates(logits, self.gate_cap, cache.states, self.matrix_state, ctx.state_slots, ctx.query_start,
                                  ctx.max_query_len, gates)
        y = ctx.buffer("matrix_memory.y", (n, H, dv), torch.float32)
        bottom = ctx.buffer("matrix_memory.bottom", (n, H), torch.float32)
        kernels.matrix_scan("memory", proj, self.q_col, proj, self.k_col, proj, self.v_col, gates, cache.states, 0,
                            ctx.state_slots, ctx.query_start, ctx.max_query_len, H, H, d, dv, y, q_scale=d ** -0.5, bottom=bottom)
        gated = ctx.buffer("matrix_memory.gated", (n, H * dv), x.dtype)
        kernels.head_norm_gate(y, bottom, self.norm_weight, proj, self.g_col, "sigmoid", self.eps, gated)
        out = ctx.buffer("matrix_memory.out", (n, self.hidden_size), x.dtype)
        kernels.linear(gated, self.o_weight, out)
        return out


@register_mixer("delta_rule")
class DeltaRule(Part):
    def __init__(self, *, prefix: str, hidden_size: int, heads: int, kv_heads: int, head_dim: int, value_dim: int, taps: int,
                 eps: float, q_name: str = "q", k_name: str = "k", v_name: str = "v", conv_suffix: str = ".conv", b_name: str = "b",
                 a_name: str = "a", a_log_name: str = "A_log", dt_bias_name: str = "dt_bias", g_name: str = "g",
                 norm_name: str = "norm", o_name: str = "o", decay_per: str = "head", decay_rank: Optional[int] = None,
                 gate_rank: Optional[int] = None, gate_activation: str = "silu") -> None:
        if min(hidden_size, heads, kv_heads, head_dim, value_dim, taps) < 1 or heads % kv_heads:
            raise ValueError(f"delta_rule: sizes must be positive and {heads} heads a multiple of {kv_heads} query/key heads")
        if head_dim > kernels.MAX_MATRIX_SCAN_DIM or taps > kernels.MAX_CONV_TAPS:
            raise ValueError(f"delta_rule: keys of {head_dim} entries (at most {kernels.MAX_MATRIX_SCAN_DIM}), {taps} taps "
                             f"(at most {kernels.MAX_CONV_TAPS})")
        self.hidden_size, self.heads, self.kv_heads = hidden_size, heads, kv_heads
        self.head_dim, self.value_dim, self.taps, self.eps = head_dim, value_dim, taps, float(eps)
        if decay_per not in ("head", "channel") or gate_activation not in kernels.HEAD_GATE_ACTIVATIONS:
            raise ValueError(f"delta_rule: decay_per {decay_per!r} (head, channel), gate_activation {gate_activation!r}")
        if decay_rank is not None and decay_per != "channel":
            raise ValueError("delta_rule: a decay projection in two steps goes with a decay per channel")
        self.decay_per, self.decay_rank, self.gate_rank = decay_per, decay_rank, gate_rank
        self.gate_activation = gate_activation
        self.decays = heads * head_dim if decay_per == "channel" else heads       # decays a token has
        qk = kv_heads * head_dim
        self.q_col, self.k_col, self.v_col = 0, qk, 2 * qk
        self.conv_channels = 2 * qk + heads * value_dim
        self.g_col = self.conv_channels
        self.conv_state = (taps - 1) * self.conv_channels
        # rows of the float32 product: the logits of beta, then the decay's logits (or its first step), then the output
        # gate's first step
        self.a_col = heads
        self.g1_col = heads + (decay_rank if decay_rank is not None else self.decays)
        self.names = {key: prefix + name for key, name in dict(
            q=q_name, k=k_name, v=v_name, q_conv=q_name + conv_suffix, k_conv=k_name + conv_suffix, v_conv=v_name + conv_suffix,
            b=b_name, a=a_name, a1=a_name + "1", a2=a_name + "2", a_log=a_log_name, dt_bias=dt_bias_name, g=g_name,
            g1=g_name + "1", g2=g_name + "2", norm=norm_name, o=o_name).items()}
        self.decay_expand = self.gate_expand = None
        self.in_weight: Optional[torch.Tensor] = None
        self.conv_weight = self.gate_weight = self.a_log = self.dt_bias = self.norm_weight = self.o_weight = None

    def param_specs(self) -> list[ParamSpec]:
        n, h, H, G, d, dv, taps = self.names, self.hidden_size, self.heads, self.kv_heads, self.head_dim, self.value_dim, self.taps
        specs = [ParamSpec(n["q"], (G * d, h)), ParamSpec(n["q_conv"], (G * d, taps)),
                 ParamSpec(n["k"], (G * d, h)), ParamSpec(n["k_conv"], (G * d, taps)),
                 ParamSpec(n["v"], (H * dv, h)), ParamSpec(n["v_conv"], (H * dv, taps)),
                 ParamSpec(n["b"], (H, h), "matrix_f32"), ParamSpec(n["a_log"], (H,), "vector"),
                 ParamSpec(n["norm"], (dv,), "vector"), ParamSpec(n["dt_bias"], (self.decays,), "vector"),
                 ParamSpec(n["o"], (h, H * dv))]
        if self.decay_rank is None:
            specs.append(ParamSpec(n["a"], (self.decays, h), "matrix_f32"))
        else:
            specs += [ParamSpec(n["a1"], (self.decay_rank, h), "matrix_f32"), ParamSpec(n["a2"], (self.decays, self.decay_rank), "matrix_f32")]
        if self.gate_rank is None:
            specs.append(ParamSpec(n["g"], (H * dv, h)))
        else:
            specs += [ParamSpec(n["g1"], (self.gate_rank, h), "matrix_f32"), ParamSpec(n["g2"], (H * dv, self.gate_rank), "matrix_f32")]
        return specs

    def cache_need(self) -> StateNeed:
        return StateNeed((self.conv_state + self.heads * self.value_dim * self.head_dim,), torch.float32)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        wide = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["g"]]] if self.gate_rank is None else [])
        self.in_weight = _pad_rows(wide, self.hidden_size)
        self.conv_weight = torch.cat([tensors[n["q_conv"]], tensors[n["k_conv"]], tensors[n["v_conv"]]], dim=0).float().contiguous()
        small = [tensors[n["b"]].float(), tensors[n["a"] if self.decay_rank is None else n["a1"]].float()]
        if self.gate_rank is not None:
            small.append(tensors[n["g1"]].float())
            self.gate_expand = tensors[n["g2"]].float().t().contiguous()          # [rank, H * dv]: the kernel reads it transposed
        if self.decay_rank is not None:
            self.decay_expand = tensors[n["a2"]].float().t().contiguous()
        self.gate_weight = torch.cat(small, dim=0).contiguous()
        self.a_log = tensors[n["a_log"]].float().contiguous()
        self.dt_bias = tensors[n["dt_bias"]].float().contiguous()
        self.norm_weight = tensors[n["norm"]].float().contiguous()
        self.o_weight = tensors[n["o"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateView) -> torch.Tensor:
        n, H, G, d, dv = x.shape[0], self.heads, self.kv_heads, self.head_dim, self.value_dim
        proj = ctx.buffer("delta_rule.proj", (n, self.in_weight.shape[0]), x.dtype)
        kernels.linear(x, self.in_weight, proj)
        logits = ctx.buffer("delta_rule.logits", (n, self.gate_weight.shape[0]), torch.float32)
        kernels.small_linear_f32(x, self.gate_weight, None, logits)
        conv = ctx.buffer("delta_rule.conv", (n, self.conv_channels), torch.float32)
        kernels.causal_conv(proj, 0, self.conv_weight, None, cache.states, 0, ctx.state_slots, ctx.query_start,
                            ctx.max_query_len, conv, activation="silu")
        kernels.unit_norm_heads(conv, self.q_col, G, d, 1e-6, d ** -0.5)
        kernels.unit_norm_heads(conv, self.k_col, G, d, 1e-6, 1.0)
        y = ctx.buffer("delta_rule.y", (n, H, dv), torch.float32)
        if self.decay_per == "channel":
            decays = ctx.buffer("delta_rule.decays", (n, H * d), torch.float32)
            if self.decay_rank is None:
                kernels.channel_decays(logits, self.a_col, self.a_log, self.dt_bias, d, decays)
            else:
                kernels.low_rank_expand(logits, self.a_col, self.decay_expand, decays, self.a_log, self.dt_bias, d)
            kernels.matrix_scan("channel_delta", conv, self.q_col, conv, self.k_col, conv, self.v_col, logits, cache.states,
                                self.conv_state, ctx.state_slots, ctx.query_start, ctx.max_query_len, H, G, d, dv, y,
                                gate_col=0, channel_decay=decays)
        else:
            gates = ctx.buffer("delta_rule.gates", (n, H, 2), torch.float32)
            kernels.decay_gates(logits, self.a_log, self.dt_bias, gates)
            kernels.matrix_scan("delta", conv, self.q_col, conv, self.k_col, conv, self.v_col, gates, cache.states, self.conv_state,
                                ctx.state_slots, ctx.query_start, ctx.max_query_len, H, G, d, dv, y)
        gated = ctx.buffer("delta_rule.gated", (n, H * dv), x.dtype)
        if self.gate_rank is None:
            gate, gate_col = proj, self.g_col
        else:
            gate, gate_col = ctx.buffer("delta_rule.gate", (n, H * dv), x.dtype), 0
            kernels.low_rank_expand(logits, self.g1_col, self.gate_expand, gate)
        kernels.head_norm_gate(y, None, self.norm_weight, gate, gate_col, self.gate_activation, self.eps, gated)
        out = ctx.buffer("delta_rule.out", (n, self.hidden_size), x.dtype)
        kernels.linear(gated, self.o_weight, out)
        return out


@register_mixer("linear_attention")
class LinearAttention(Part):
    def __init__(self, *, prefix: str, hidden_size: int, heads: int, head_dim: int, value_dim: int, decay, eps: float,
                 q_name: str = "q", k_name: str = "k", v_name: str = "v", g_name: str = "g", o_name: str = "o",
                 norm_name: str = "norm") -> None:
        decay = tuple(float(value) for value in decay)
        if min(hidden_size, heads, head_dim, value_dim) < 1 or len(decay) != heads:
            raise ValueError(f"linear_attention: sizes must be positive, and {len(decay)} decays were given for {heads} heads")
        if head_dim > kernels.MAX_MATRIX_SCAN_DIM:
            raise ValueError(f"linear_attention: keys of {head_dim} entries exceed {kernels.MAX_MATRIX_SCAN_DIM}")
        self.hidden_size, self.heads, self.head_dim, self.value_dim, self.eps = hidden_size, heads, head_dim, value_dim, float(eps)
        self.decay = decay
        self.q_col, self.k_col, self.v_col = 0, heads * head_dim, 2 * heads * head_dim
        self.g_col = self.v_col + heads * value_dim
        self.names = {key: prefix + name for key, name in dict(q=q_name, k=k_name, v=v_name, g=g_name, o=o_name, norm=norm_name).items()}
        self.in_weight = self.norm_weight = self.o_weight = self.decay_on_device = None

    def param_specs(self) -> list[ParamSpec]:
        n, h, H, d, dv = self.names, self.hidden_size, self.heads, self.head_dim, self.value_dim
        return [ParamSpec(n["q"], (H * d, h)), ParamSpec(n["k"], (H * d, h)), ParamSpec(n["v"], (H * dv, h)),
                ParamSpec(n["g"], (H * dv, h)), ParamSpec(n["o"], (h, H * dv)), ParamSpec(n["norm"], (H * dv,), "vector")]

    def cache_need(self) -> StateNeed:
        return StateNeed((self.heads * self.value_dim * self.head_dim,), torch.float32)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        n = self.names
        self.in_weight = _pad_rows([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]]], self.hidden_size)
        self.norm_weight = tensors[n["norm"]].float().contiguous()
        self.o_weight = tensors[n["o"]]
        self.decay_on_device = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(self.o_weight.device)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateView) -> torch.Tensor:
        n, H, d, dv = x.shape[0], self.heads, self.head_dim, self.value_dim
        proj = ctx.buffer("linear_attention.proj", (n, self.in_weight.shape[0]), x.dtype)
        kernels.linear(x, self.in_weight, proj)
        y = ctx.buffer("linear_attention.y", (n, H, dv), torch.float32)
        kernels.matrix_scan("decay", proj, self.q_col, proj, self.k_col, proj, self.v_col, self.decay_on_device, cache.states, 0,
                            ctx.state_slots, ctx.query_start, ctx.max_query_len, H, H, d, dv, y, input_activation="silu")
        gated = ctx.buffer("linear_attention.gated", (n, H * dv), x.dtype)
        # (the heads are normed together: one "head" of H * dv entries)
        kernels.head_norm_gate(y.view(n, 1, H * dv), None, self.norm_weight, proj, self.g_col, "sigmoid", self.eps, gated)
        out = ctx.buffer("linear_attention.out", (n, self.hidden_size), x.dtype)
        kernels.linear(gated, self.o_weight, out)
        return out
