"""The gated linear recurrence mixer (``gated_linear_recurrence``): the recurrent block of the Griffin family, a
real-gated linear recurrent unit behind a short convolution.

With ``h`` the input and ``W`` channels in ``B`` equal parts:

* two branches, ``y = gelu_tanh(W_y h + b_y)`` and ``u = conv(W_x h + b_x)``, a causal convolution per channel with a bias
  and no activation (zeros before the start of a sequence: the projection's bias is part of the convolution's input);
* in each part ``b`` the gates ``r = sigmoid(R_b u_b + c_b)`` and ``i = sigmoid(I_b u_b + e_b)`` with square matrices ``R_b``,
  ``I_b``;
* ``log a = -8 r softplus(lam)``, ``S_t = a S_(t-1) + sqrt(1 - a^2) i u`` from ``S = 0``, and the output ``W_o (S y)``.

What a request carries from token to token is one float32 vector per layer (:class:`~.base.StateNeed`, zero at
admission): the convolution's last ``taps - 1`` inputs, then ``S``.  The convolution, the gates (their block-diagonal
products included), the decay and the recurrence are float32 whatever the compute type; the two wide projections are in
the compute type.  ``gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))``.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, StateNeed, register_mixer
from .context import StateView, StepContext

DECAY_SHARPNESS = 8.0      # log a = -DECAY_SHARPNESS * r * softplus(lam)


@register_mixer("gated_linear_recurrence")
class GatedLinearRecurrence(Part):
    def __init__(self, *, prefix: str, hidden_size: int, width: int, blocks: int, taps: int, y_name: str = "y",
                 y_bias_name: str = "y.b", x_name: str = "x", x_bias_name: str = "x.b", conv_name: str = "conv",
                 conv_bias_name: str = "conv.b", r_name: str = "ra", r_bias_name: str = "ra.b", i_name: str = "ri",
                 i_bias_name: str = "ri.b", lam_name: str = "lam", o_name: str = "o") -> None:
        if min(hidden_size, width, blocks, taps) < 1 or width % blocks or taps > kernels.MAX_CONV_TAPS:
            raise ValueError(f"gated_linear_recurrence: {width} channels in {blocks} parts, {taps} taps (at most {kernels.MAX_CONV_TAPS})")
        self.hidden_size, self.width, self.blocks, self.taps = hidden_size, width, blocks, taps
        self.part = width // blocks
        self.in_rows = (2 * width + 7) // 8 * 8
        self.conv_state = (taps - 1) * width
        self.names = {key: prefix + name for key, name in dict(
            y=y_name, y_b=y_bias_name, x=x_name, x_b=x_bias_name, conv=conv_name, conv_b=conv_bias_name, r=r_name,
            r_b=r_bias_name, i=i_name, i_b=i_bias_name, lam=lam_name, o=o_name).items()}
        self.in_weight: Optional[torch.Tensor] = None
        self.in_bias = self.conv_weight = self.conv_bias = self.gate_weight = self.gate_bias = self.rate = self.o_weight = None

    def param_specs(self) -> list[ParamSpec]:
        n, h, w, b, p = self.names, self.hidden_size, self.width, self.blocks, self.part
        return [ParamSpec(n["y"], (w, h)), ParamSpec(n["y_b"], (w,), "vector"), ParamSpec(n["x"], (w, h)),
                ParamSpec(n["x_b"], (w,), "vector"), ParamSpec(n["conv"], (w, self.taps)), ParamSpec(n["conv_b"], (w,), "vector"),
                ParamSpec(n["r"], (b, p, p), "matrix_f32"), ParamSpec(n["r_b"], (b, p), "vector"),
                ParamSpec(n["i"], (b, p, p), "matrix_f32"), ParamSpec(n["i_b"], (b, p), "vector"),
                ParamSpec(n["lam"], (w,), "vector"), ParamSpec(n["o"], (h, w))]

    def cache_need(self) -> StateNeed:
        return StateNeed((self.conv_state + self.width,), torch.float32)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        n, w = self.names, self.width
        pieces = [tensors[n["y"]], tensors[n["x"]]]
        padding = self.in_rows - 2 * w
        if padding:
            pieces.append(torch.zeros((padding, self.hidden_size), dtype=pieces[0].dtype, device=pieces[0].device))
        self.in_weight = torch.cat(pieces, dim=0).contiguous()
        self.in_bias = torch.cat([tensors[n["y_b"]].float(), tensors[n["x_b"]].float()]).contiguous()       # [y | x]
        self.conv_weight = tensors[n["conv"]].float().contiguous()
        self.conv_bias = tensors[n["conv_b"]].float().contiguous()
        self.gate_weight = torch.stack([tensors[n["r"]].float(), tensors[n["i"]].float()]).contiguous()       # [2, B, p, p]
        self.gate_bias = torch.stack([tensors[n["r_b"]].float().reshape(w), tensors[n["i_b"]].float().reshape(w)]).contiguous()
        # log a = rate * r with rate = -8 softplus(lam), formed once in float32
        self.rate = (-DECAY_SHARPNESS * torch.nn.functional.softplus(tensors[n["lam"]].float())).contiguous()
        self.o_weight = tensors[n["o"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateView) -> torch.Tensor:
        n, w, b, p = x.shape[0], self.width, self.blocks, self.part
        proj = ctx.buffer("linear_recurrence.proj", (n, self.in_rows), x.dtype)
        kernels.linear(x, self.in_weight, proj)
        u = ctx.buffer("linear_recurrence.u", (n, w), torch.float32)
        kernels.causal_conv(proj, w, self.conv_weight, self.conv_bias, cache.states, 0, ctx.state_slots, ctx.query_start,
                            ctx.max_query_len, u, activation="none", in_bias=self.in_bias[w:])
        pre = ctx.buffer("linear_recurrence.pre", (2, n, w), torch.float32)
        parts = u.view(n, b, p).transpose(0, 1)                       # [B, n, p]: part b's columns of every row
        for gate in range(2):
            kernels.linear_batched(parts, self.gate_weight[gate], pre[gate].view(n, b, p).transpose(0, 1))
        gated = ctx.buffer("linear_recurrence.gated", (n, w), x.dtype)
        kernels.gated_recurrence_scan(u, pre, self.gate_bias, self.rate, proj, 0, self.in_bias[:w], cache.states,
                                      self.conv_state, ctx.state_slots, ctx.query_start, ctx.max_query_len, gated)
        out = ctx.buffer("linear_recurrence.out", (n, self.hidden_size), x.dtype)
        kernels.linear(gated, self.o_weight, out)
        return out
