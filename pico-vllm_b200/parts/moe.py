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
after the experts' own, experts without tensors whose output is their input (times the weight).

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

_ACTS = {"silu": ops.MOE_ACT_SILU, "relu2": ops.MOE_ACT_RELU2}
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
                 shared_inner: Optional[int] = None, choice_bias: bool = False, weight_scale: float = 1.0, identity: int = 0):
        if act not in _ACTS or (gated and act != "silu"):
            raise ConfigError(f"routed_experts: activation {act!r} is not built (gated: 'silu'; not gated: {sorted(_ACTS)})")
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
            ps += [Param("shared_up_weight", tuple(self._up_pieces("shared.", self.shared_inner))),
                   Param("shared_down_weight", (Piece("shared.down.weight", (self.width, self.shared_inner)),))]
        return ps

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "gate_up_weight":
            tensor = tensor.view(self.experts, (2 if self.gated else 1) * self.inner, self.width)
        elif attr == "down_weight":
            tensor = tensor.view(self.experts, self.width, self.inner)
        setattr(self, attr, tensor)

    def _shared(self, h: torch.Tensor) -> torch.Tensor:
        """The shared expert: two plain products with the activation between them."""
        u = _linear(h, self.shared_up_weight)
        if self.gated:
            a = torch.empty((h.shape[0], self.shared_inner), dtype=h.dtype, device=h.device)
            ops.swiglu(u, a)
        else:
            a = ops.activation(u, self.act)
        return _linear(a, self.shared_down_weight)

    def forward(self, h: torch.Tensor, batch) -> torch.Tensor:
        base = self._shared(h) if self.shared_inner else None
        idx, wgt = ops.moe_route(h, self.router_weight, self.router_bias, self.top, self.scoring, self.choice_bias,
                                 self.weight_scale)
        return ops.moe_experts(h, idx, wgt, self.gate_up_weight, self.down_weight, gated=self.gated, act=self.act,
                               weight_on_input=self.weight_on == "input", base=base, identity=self.identity)
