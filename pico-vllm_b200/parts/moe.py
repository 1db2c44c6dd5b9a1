"""Routed experts: every token goes through ``top`` of ``experts`` small feed-forwards.

The default form (gated experts, softmax over the chosen logits, the weight on the expert's output):

    z = W_r h + b_r  (float32)        chosen = the top largest z        weight = softmax over the chosen z alone
    y = sum over chosen e of weight_e * W_down[e] ( silu(W_gate[e] h) * (W_up[e] h) )

Options, each a constructor argument: ``gated=False`` - an expert is W_down act(W_up h) with ``act`` "silu" or "relu2"
(the square of relu); ``scoring="sigmoid"`` - the weight of a chosen expert is sigmoid(z_e), not renormalised (the choice
is still the largest z); ``weight_on="input"`` - the weight multiplies what the expert reads, y = sum_e expert_e(weight_e
h), not what it returns; ``shared_inner`` - one more expert of the same form and that inner size which every token goes
through with weight 1 and whose output is added; ``scoring="softmax_all"`` - an expert's score is its share of the softmax
over ALL router outputs, the choice is by score + a learned ``choice_bias`` (``choice_bias=True``: tensor ``correction``),
the weight is the score itself times ``weight_scale``, not renormalised; ``identity`` n - the router has n more outputs
after the experts' own, experts without tensors whose output is their input (times the weight); ``groups`` /
``groups_keep`` - the experts form ``groups`` equal runs of neighbours and only experts of the ``groups_keep`` runs whose
best score + choice bias is largest can be chosen; ``renorm`` - the weights are the chosen scores divided by their sum
(+ 1e-20), then times ``weight_scale``; ``act="capped"`` with ``limit`` L - a gated expert is W_down (g' sigmoid(1.702 g')
(u' + 1)) with g' = min(W_gate h, L), u' = clamp(W_up h, -L, L); ``shared_limit`` - the shared expert's own L;
``shared_gate`` - the shared expert's output is multiplied by sigmoid(w_sg . h), one number a token (tensor ``shared.sg``).

Router, choice, listing of tokens per expert, both products (grouped over the experts' token lists) and the sum run on
the device without a look from the host.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..errors import ConfigError
from .base import Param, Part, Piece
from .registry import register

_ACTS = {"silu": ops.MOE_ACT_SILU, "relu2": ops.MOE_ACT_RELU2, "capped": ops.MOE_ACT_CAPPED}
_SCORINGS = {"softmax_chosen": ops.MOE_SCORE_SOFTMAX_CHOSEN, "sigmoid": ops.MOE_SCORE_SIGMOID,
             "softmax_all": ops.MOE_SCORE_SOFTMAX_ALL}


def _linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if ops.skinny_takes(x, weight):
        return ops.skinny_linear(x, weight)
    return ops.linear(x, weight)


@register("feed_forward", "routed_experts")
class RoutedExperts(Part):
    def __init__(self, width: int, inner: int, experts: int, top: int, act: str = "silu", router_bias: bool = True,
                 gated: bool = True, scoring: str = "softmax_chosen", weight_on: str = "output",
                 shared_inner: Optional[int] = None, choice_bias: bool = False, weight_scale: float = 1.0, identity: int = 0,
                 groups: int = 1, groups_keep: int = 1, renorm: bool = False, limit: Optional[float] = None,
                 shared_limit: Optional[float] = None, shared_gate: bool = False):
        if act not in _ACTS or (gated and act not in ("silu", "capped")) or (act == "capped" and not gated):
            raise ConfigError(f"routed_experts: activation {act!r} is not built (gated: 'silu', 'capped'; not gated: 'silu', 'relu2')")
        if act == "capped" and not (limit and limit > 0 and (not shared_inner or (shared_limit or limit) > 0)):
            raise ConfigError("routed_experts: the capped activation needs a positive limit")
        if (groups != 1 or renorm) and scoring != "softmax_all":
            raise ConfigError("routed_experts: expert groups and renormalised weights are built for scoring 'softmax_all'")
        if groups < 1 or (experts + identity) % groups or not 1 <= groups_keep <= groups \
                or top > (experts + identity) // groups * groups_keep:
            raise ConfigError(f"routed_experts: {experts + identity} experts in {groups} groups of which {groups_keep} stay cannot give {top} choices")
        if shared_gate and not (shared_inner and act == "capped"):
            raise ConfigError("routed_experts: a gate on the shared expert is built for a shared expert of the capped form")
        if scoring not in _SCORINGS:
            raise ConfigError(f"routed_experts: scoring {scoring!r} is not built (have {sorted(_SCORINGS)})")
        if weight_on not in ("output", "input") or (gated and weight_on == "input"):
            raise ConfigError("routed_experts: weight_on must be 'output', or 'input' for experts without a gate")
        if identity < 0 or (identity and weight_on != "output"):
            raise ConfigError("routed_experts: experts that hand their input on are built with the weight on the output")
        if (choice_bias or weight_scale != 1.0) and scoring != "softmax_all":
            raise ConfigError("routed_experts: a choice bias and a weight scale are built for scoring 'softmax_all'")
        if not 1 <= top <= experts + identity or top > 32:
            raise ConfigError(f"routed_experts: top {top} must lie in 1..min(experts, 32) (experts: {experts + identity})")
        self.width, self.inner, self.experts, self.top, self.has_bias = width, inner, experts, top, router_bias
        self.gated, self.act, self.scoring, self.weight_on = gated, _ACTS[act], _SCORINGS[scoring], weight_on
        self.shared_inner = shared_inner
        self.has_choice_bias, self.weight_scale, self.identity = choice_bias, float(weight_scale), identity
        self.groups, self.groups_keep, self.renorm = groups, groups_keep, renorm
        self.limit = float(limit) if limit else 0.0
        self.shared_limit = float(shared_limit) if shared_limit else self.limit
        self.shared_gate = shared_gate
        self.choice_bias = None
        self.router_weight = self.router_bias = self.gate_up_weight = self.down_weight = None
        self.shared_up_weight = self.shared_down_weight = None

    def _up_pieces(self, prefix: str, inner: int) -> List[Piece]:
        ups = [Piece(f"{prefix}gate.weight", (inner, self.width))] if self.gated else []
        return ups + [Piece(f"{prefix}up.weight", (inner, self.width))]

    def params(self) -> List[Param]:
        gate_up, down = [], []
        for e in range(self.experts):
            gate_up += self._up_pieces(f"e{e}.", self.inner)
            down.append(Piece(f"e{e}.down.weight", (self.width, self.inner)))
        ps = [Param("router_weight", (Piece("router.weight", (self.experts + self.identity, self.width)),), kind="vector"),
              Param("gate_up_weight", tuple(gate_up)), Param("down_weight", tuple(down))]
        if self.has_bias:
            ps.append(Param("router_bias", (Piece("router.bias", (self.experts,)),), kind="vector"))
        if self.has_choice_bias:
            ps.append(Param("choice_bias", (Piece("correction", (self.experts + self.identity,)),), kind="vector"))
        if self.shared_inner:
            ups = self._up_pieces("shared.", self.shared_inner)
            if self.shared_gate:
                ups.append(Piece("shared.sg.weight", (1, self.width)))
            ps += [Param("shared_up_weight", tuple(ups)),
                   Param("shared_down_weight", (Piece("shared.down.weight", (self.width, self.shared_inner)),))]
        return ps

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "gate_up_weight":
            tensor = tensor.view(self.experts, (2 if self.gated else 1) * self.inner, self.width)
        elif attr == "down_weight":
            tensor = tensor.view(self.experts, self.width, self.inner)
        elif attr == "shared_up_weight" and self.shared_gate and tensor.shape[0] % 16:    # the gate's one row: padded to the next multiple of 16 rows
            tensor = torch.cat([tensor, tensor.new_zeros((16 - tensor.shape[0] % 16, tensor.shape[1]))], 0).contiguous()
        setattr(self, attr, tensor)

    def _shared(self, h: torch.Tensor) -> torch.Tensor:
        """The shared expert: two plain products with the activation between them."""
        u = _linear(h, self.shared_up_weight)
        if self.act == ops.MOE_ACT_CAPPED:
            n = (2 if self.gated else 1) * self.shared_inner
            a = ops.capped_glu(u, self.shared_inner, self.shared_limit, n if self.shared_gate else None)
        elif self.gated:
            a = torch.empty((h.shape[0], self.shared_inner), dtype=h.dtype, device=h.device)
            ops.swiglu(u, a)
        else:
            a = ops.activation(u, self.act)
        return _linear(a, self.shared_down_weight)

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        base = self._shared(h) if self.shared_inner else None
        idx, wgt = ops.moe_route(h, self.router_weight, self.router_bias, self.top, self.scoring, self.choice_bias,
                                 self.weight_scale, self.groups, self.groups_keep, self.renorm)
        return ops.moe_experts(h, idx, wgt, self.gate_up_weight, self.down_weight, gated=self.gated, act=self.act,
                               weight_on_input=self.weight_on == "input", base=base, identity=self.identity, limit=self.limit)
