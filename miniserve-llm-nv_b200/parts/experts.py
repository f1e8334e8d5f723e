"""A feed-forward of routed experts (``routed_experts``).

``experts`` small feed-forward layers without biases, of which every token uses ``top``:

* router logits ``z = W_r h + b`` in float32 (the router's weight and bias are kept in float32);
* the ``top`` experts with the largest logits are chosen (a tie goes to the lower index), and their weights are the
  softmax over the chosen logits alone;
* expert ``e`` computes ``W_down,e act(W_up,e h)``; the output is the weighted sum of the chosen experts' outputs;
* a shared expert of the same form (its own inner size), if any, runs for every token and is added.

``activation``: ``relu_square`` (``act(z) = max(z, 0)^2`` of one up projection), or ``clamped_glu``: an expert has a
gate and an up projection, ``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``, and
``y = g sigmoid(1.702 g) (u + 1)`` enters the down projection (the two weights are kept as one whose rows alternate,
gate row j, up row j, so that one product's epilogue holds both).  The shared expert has the same form with
``shared_limit``.  ``silu_glu``: ``y = silu(W_gate h) (W_up h)``, the same two weights kept the same way, no limit.

Other ways to route, each off by default:

* ``scoring="all_softmax"``: scores are the softmax over ALL router outputs, and a chosen expert's weight is its score
  as it is (the weights of a token then do not add up to 1).  ``correction_name``: a vector added to the scores for the
  CHOICE only.
* ``groups=(count, keep)``: the router's outputs form ``count`` equal groups of neighbours; a group's score is its
  largest choice score, and only members of the ``keep`` best groups can be chosen.
* ``scoring="sigmoid"``: scores are ``sigmoid(z)`` of every router output on its own; the ``top`` largest are chosen (a tie
  goes to the lower index) and a chosen expert's weight is its score as it is.
* ``weight_on="input"``: the weight multiplies what the expert reads, not what it returns: the output is the sum of
  ``expert(w h)`` over the chosen experts.  (An expert's first products are linear, so the factor is applied to their
  float32 sums as the activation is formed.)
* ``identity``: the last ``identity`` router outputs stand for experts without tensors whose output is their input.
* ``shared_gate_name``: a ``[1, width]`` weight; the shared expert's output is multiplied by ``sigmoid(w . h)`` per
  token (the row rides along with the router's float32 product).

Everything happens on the device, so a step never waits for the host to learn the choice and a captured decode
step can hold the layer: the (token, choice) pairs are sorted by expert (``kernels.expert_route``), each expert's
two products run over its segment of rows (``kernels.expert_linear``, the first gathering its rows from the tokens and
applying the activation as it stores), and one kernel adds a token's weighted results and the shared expert's
(``kernels.expert_combine``, float32 sums).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, register_feed_forward
from .context import StepContext


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    def __init__(self, *, prefix: str, hidden_size: int, experts: int, top: int, expert_size: int,
                 shared_size: Optional[int] = None, router_bias: bool = True, activation: str = "relu_square",
                 router_name: str = "router", router_bias_name: str = "router.b", expert_name: str = "e{index}.",
                 shared_name: str = "shared.", up_name: str = "up", down_name: str = "down", gate_name: str = "gate",
                 limit: Optional[float] = None, shared_limit: Optional[float] = None, identity: int = 0,
                 scoring: str = "chosen_softmax", correction_name: Optional[str] = None, groups: tuple = (1, 1),
                 shared_gate_name: Optional[str] = None, weight_on: str = "output") -> None:
        if activation not in ("relu_square", "clamped_glu", "silu_glu"):
            raise ValueError(f"routed_experts implements the activations 'relu_square', 'clamped_glu' and 'silu_glu', not {activation!r}")
        if scoring not in ("chosen_softmax", "all_softmax", "sigmoid"):
            raise ValueError(f"routed_experts scores by 'chosen_softmax', 'all_softmax' or 'sigmoid', not {scoring!r}")
        if weight_on not in ("output", "input"):
            raise ValueError(f"routed_experts weights an expert's 'output' or its 'input', not {weight_on!r}")
        if weight_on == "input" and (activation != "silu_glu" or identity):
            raise ValueError("weights on the experts' inputs are implemented for the 'silu_glu' activation without identity experts")
        total = experts + identity
        count, keep = (int(g) for g in groups)
        if identity < 0 or count < 1 or total % count or not 1 <= keep <= count:
            raise ValueError(f"{total} router outputs ({identity} identities) in {count} groups of which {keep} are kept: not possible")
        if not 1 <= top <= keep * (total // count):
            raise ValueError(f"every token uses {top} of {total} experts ({keep} of {count} groups kept): not possible")
        if activation == "clamped_glu" and (limit is None or (shared_size and shared_limit is None)):
            raise ValueError("the clamped activation needs its limit (and the shared expert's)")
        if activation == "silu_glu" and shared_size:
            raise ValueError("a shared expert is not implemented for the 'silu_glu' activation")
        if (correction_name or (count, keep) != (1, 1)) and scoring not in ("all_softmax", "sigmoid"):
            raise ValueError("a correction of the choice and groups are implemented for scoring='all_softmax'")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.experts, self.top, self.expert_size, self.shared_size = experts, top, expert_size, shared_size
        self.identity, self.total, self.scoring, self.groups = identity, total, scoring, (count, keep)
        self.gated = activation in ("clamped_glu", "silu_glu")
        self.activation, self.weight_on = activation, weight_on
        self.limit = float(limit) if limit is not None else 0.0
        self.shared_limit = float(shared_limit) if shared_limit is not None else 0.0
        self.router_bias = bool(router_bias)
        self.names = dict(router=prefix + router_name, bias=prefix + router_bias_name,
                          up=[prefix + expert_name.format(index=e) + up_name for e in range(experts)],
                          gate=[prefix + expert_name.format(index=e) + gate_name for e in range(experts)],
                          down=[prefix + expert_name.format(index=e) + down_name for e in range(experts)],
                          shared_up=prefix + shared_name + up_name, shared_gate_proj=prefix + shared_name + gate_name,
                          shared_down=prefix + shared_name + down_name,
                          correction=None if correction_name is None else prefix + correction_name,
                          shared_gate=None if shared_gate_name is None or not shared_size else prefix + shared_gate_name)
        self.correction: Optional[torch.Tensor] = None       # float32 [total]
        self.router_weight: Optional[torch.Tensor] = None    # float32 [E, hidden]
        self.router_b: Optional[torch.Tensor] = None         # float32 [E]
        self.up: Optional[torch.Tensor] = None               # [E, expert_size, hidden]
        self.down: Optional[torch.Tensor] = None             # [E, hidden, expert_size]
        self.shared_up: Optional[torch.Tensor] = None
        self.shared_down: Optional[torch.Tensor] = None

    def param_specs(self) -> list[ParamSpec]:
        h, names = self.hidden_size, self.names
        specs = []
        for e in range(self.experts):
            if self.gated:
                specs.append(ParamSpec(names["gate"][e], (self.expert_size, h)))
            specs += [ParamSpec(names["up"][e], (self.expert_size, h)), ParamSpec(names["down"][e], (h, self.expert_size))]
        specs.append(ParamSpec(names["router"], (self.total, h), "matrix_f32"))
        if self.router_bias:
            specs.append(ParamSpec(names["bias"], (self.total,), "vector"))
        if names["correction"]:
            specs.append(ParamSpec(names["correction"], (self.total,), "vector"))
        if self.shared_size:
            if self.gated:
                specs.append(ParamSpec(names["shared_gate_proj"], (self.shared_size, h)))
            specs += [ParamSpec(names["shared_up"], (self.shared_size, h)), ParamSpec(names["shared_down"], (h, self.shared_size))]
        if names["shared_gate"]:
            specs.append(ParamSpec(names["shared_gate"], (1, h), "matrix_f32"))
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        names = self.names
        router = tensors[names["router"]].float()
        if names["shared_gate"]:
            # the shared expert's gate logit is one more row of the router's float32 product
            router = torch.cat([router, tensors[names["shared_gate"]].float().view(1, -1)], dim=0)
        self.router_weight = router.contiguous()
        self.router_b = tensors[names["bias"]].float().contiguous() if self.router_bias else None
        if self.router_b is not None and names["shared_gate"]:
            self.router_b = torch.cat([self.router_b, torch.zeros_like(self.router_b[:1])]).contiguous()
        self.correction = tensors[names["correction"]].float().contiguous() if names["correction"] else None

        def alternate(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
            return torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1])

        if self.gated:
            self.up = torch.stack([alternate(tensors[g], tensors[u]) for g, u in zip(names["gate"], names["up"])]).contiguous()
        else:
            self.up = torch.stack([tensors[name] for name in names["up"]]).contiguous()
        self.down = torch.stack([tensors[name] for name in names["down"]]).contiguous()
        if self.shared_size:
            self.shared_up, self.shared_down = tensors[names["shared_up"]], tensors[names["shared_down"]]
            if self.gated:
                self.shared_up = alternate(tensors[names["shared_gate_proj"]], self.shared_up).contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        n, top, width = x.shape[0], self.top, self.hidden_size
        pairs = n * top
        ids = ctx.buffer("experts.ids", (n, top), torch.int32)
        weights = ctx.buffer("experts.weights", (n, top), torch.float32)
        logits = ctx.buffer("experts.logits", (n, self.router_weight.shape[0]), torch.float32)
        kernels.router_topk(x, self.router_weight, self.router_b, top, ids, weights, logits, choose_from=self.total,
                            scoring=self.scoring, correction=self.correction, groups=self.groups)
        offsets = ctx.buffer("experts.offsets", (self.total + 1,), torch.int32)
        order = ctx.buffer("experts.order", (pairs,), torch.int32)
        place = ctx.buffer("experts.place", (pairs,), torch.int32)
        kernels.expert_route(ids, self.total, offsets, order, place)
        # (the segments of identity experts lie behind those of the experts with tensors; their rows are not computed)
        hidden = ctx.buffer("experts.hidden", (pairs, self.expert_size), x.dtype)
        if self.gated:
            kernels.expert_linear(x, order, top, self.up, hidden, offsets, activation=self.activation, limit=self.limit,
                                  pair_scale=weights if self.weight_on == "input" else None)
        else:
            kernels.expert_linear(x, order, top, self.up, hidden, offsets, activation="relu_square")
        results = ctx.buffer("experts.results", (pairs, width), x.dtype)
        kernels.expert_linear(hidden, None, top, self.down, results, offsets)
        shared = None
        if self.shared_size:
            shared_hidden = ctx.buffer("experts.shared_hidden", (n, self.shared_size), x.dtype)
            if self.gated:
                both = ctx.buffer("experts.shared_both", (n, 2 * self.shared_size), x.dtype)
                kernels.linear(x, self.shared_up, both)
                kernels.clamped_glu(both, self.shared_limit, shared_hidden)
            else:
                kernels.linear(x, self.shared_up, shared_hidden)
                kernels.relu_square(shared_hidden)
            shared = ctx.buffer("experts.shared", (n, width), x.dtype)
            kernels.linear(shared_hidden, self.shared_down, shared)
        out = ctx.buffer("experts.out", (n, width), x.dtype)
        kernels.expert_combine(results, place, None if self.weight_on == "input" else weights, shared, out, ids=ids if self.identity else None,
                               first_identity=self.experts, x=x if self.identity else None,
                               shared_gate=logits if self.names["shared_gate"] else None, shared_gate_col=self.total)
        return out
