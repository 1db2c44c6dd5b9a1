"""Norms on the float32 residual stream, fused with the residual add that precedes them.

:class:`RMSNorm` and :class:`CentredNorm` (mean taken off, weight, no bias).  What is added may itself be normed
first (:class:`NormedDelta`: a sublayer's output with the norm that stands between it and the stream): norm,
add and the next norm are then one kernel.

y = x * rsqrt(mean(x^2) + eps) * w in float32 (pico_vllm/RMSNorm.py:22-34; plain form
pico_vllm/model.py:57-66).  The reference adds the residual in a separate torch op
(pico_vllm/model.py:372-373); here the add and the norm are one kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Union

import torch

from .. import ops
from .base import Param, Part, Piece
from .registry import register


@dataclass
class NormedDelta:
    """A sublayer's output that is still to pass through ``norm`` before it is added to the residual stream."""
    delta: torch.Tensor
    norm: "Part"


@dataclass
class SumDelta:
    """Several sublayer outputs that are still to be added to the residual stream together: ``terms`` is a list of
    (delta, norm or None, scale) - each passes through its own norm (an RMS norm with a weight) or none and is multiplied
    by ``scale`` on its way.  Up to three terms."""
    terms: list

    def flat(self):
        return [(d, None if n is None else n.weight, ops.NORM_NONE if n is None else n.norm_kind, 0.0 if n is None else n.eps, s)
                for d, n, s in self.terms]


def _sum_add_norm(norm, kind: int, x: torch.Tensor, delta: "SumDelta", rows: Optional[torch.Tensor]) -> torch.Tensor:
    if norm.act_dtype == torch.float32 and kind == ops.NORM_COPY and rows is None:
        ops.sum_add_norm(x, delta.flat(), None, ops.NORM_NONE, 0.0, None)
        return x                         # in float32 the stream itself is handed on (readers must not write to it)
    n = rows.shape[0] if rows is not None else x.shape[0]
    out = torch.empty((n, norm.width), dtype=norm.act_dtype, device=x.device)
    return ops.sum_add_norm(x, delta.flat(), norm.weight, kind, norm.eps, out, rows)


def _post_add_norm(norm, kind: int, x: torch.Tensor, delta, rows: Optional[torch.Tensor]) -> torch.Tensor:
    n = rows.shape[0] if rows is not None else x.shape[0]
    out = torch.empty((n, norm.width), dtype=norm.act_dtype, device=x.device)
    post = None
    if isinstance(delta, NormedDelta):
        post, delta = delta.norm, delta.delta
    return ops.post_add_norm(x, delta, None if post is None else post.weight, 0 if post is None else post.norm_kind,
                             0.0 if post is None else post.eps, norm.weight, kind, norm.eps, out, rows)


@register("norm", "rmsnorm")
class RMSNorm(Part):
    # y = x * rsqrt(mean(x^2) + eps) * weight and nothing else: what the product kernels with the norm inside
    # compute.  A part that takes a norm into its own kernel asks for this mark, not for attribute names.
    plain_rms = True
    norm_kind = ops.NORM_RMS

    def __init__(self, width: int, eps: float, one_plus: bool = False):
        """``one_plus``: the stored tensor lies around zero and the norm multiplies by 1 + it (added once, in float32,
        when the tensor is loaded; the kernels see an ordinary weight)."""
        self.width, self.eps, self.one_plus = width, eps, one_plus
        self.weight: Optional[torch.Tensor] = None
        self.act_dtype = torch.bfloat16

    def params(self) -> List[Param]:
        return [Param("weight", (Piece("weight", (self.width,)),), kind="vector",
                      init="normal" if self.one_plus else "one_plus_normal")]

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "weight" and self.one_plus:
            tensor = tensor.to(torch.float32) + 1.0
        setattr(self, attr, tensor)

    def materialize(self, device, dtype):
        self.act_dtype = dtype

    def add_norm(self, x: torch.Tensor, delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: float32 [T, width] residual stream, updated in place by ``x += delta`` unless
        ``rows`` picks rows (then x stays).  Returns norm(x) in the activation dtype."""
        if x.dim() == 3:                # several residual streams [T, S, width]: what is read is their sum
            from .hyper import streams_add_norm
            return streams_add_norm(self, x, delta, None, rows)
        if isinstance(delta, NormedDelta):
            return _post_add_norm(self, ops.NORM_RMS, x, delta, rows)
        if isinstance(delta, SumDelta):
            return _sum_add_norm(self, ops.NORM_RMS, x, delta, rows)
        n = rows.shape[0] if rows is not None else x.shape[0]
        out = torch.empty((n, self.width), dtype=self.act_dtype, device=x.device)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)


@register("norm", "scalar_rmsnorm")
class ScalarRMSNorm(RMSNorm):
    """y = x * rsqrt(mean(x^2) + eps) * g with ONE learned number g for all coordinates.  The number is spread over a
    vector when it is loaded, so the kernels see an ordinary RMS norm."""

    def __init__(self, width: int, eps: float):
        super().__init__(width, eps, one_plus=False)

    def params(self) -> List[Param]:
        return [Param("weight", (Piece("weight", ()),), kind="vector", init="one_plus_normal")]

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "weight":
            tensor = tensor.to(torch.float32).reshape(1).expand(self.width).contiguous()
        setattr(self, attr, tensor)


@register("norm", "centred_norm")
class CentredNorm(Part):
    """y = (x - mean x) / sqrt(mean((x - mean x)^2) + eps) * weight: a layer norm with a weight and no bias,
    float32 throughout."""
    norm_kind = ops.NORM_CENTRED

    def __init__(self, width: int, eps: float):
        self.width, self.eps = width, eps
        self.weight: Optional[torch.Tensor] = None
        self.act_dtype = torch.bfloat16

    def params(self) -> List[Param]:
        return [Param("weight", (Piece("weight", (self.width,)),), kind="vector", init="one_plus_normal")]

    def materialize(self, device, dtype):
        self.act_dtype = dtype

    def add_norm(self, x: torch.Tensor, delta: Union[None, torch.Tensor, NormedDelta],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """As :meth:`RMSNorm.add_norm`; ``delta`` may be a :class:`NormedDelta`."""
        return _post_add_norm(self, ops.NORM_CENTRED, x, delta, rows)


@register("norm", "none")
class PassNorm(Part):
    """No norm at all: ``add_norm`` adds what is pending to the residual stream and hands the stream on in the
    activation type - the input norm of a layer whose sublayers read the stream itself.  In float32 the stream is
    handed on as it is (readers must not write to it)."""
    norm_kind = ops.NORM_COPY
    weight = None
    eps = 0.0

    def __init__(self, width: int):
        self.width = width
        self.act_dtype = torch.bfloat16

    def materialize(self, device, dtype):
        self.act_dtype = dtype

    def add_norm(self, x: torch.Tensor, delta: Union[None, torch.Tensor, NormedDelta],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if isinstance(delta, SumDelta):
            return _sum_add_norm(self, ops.NORM_COPY, x, delta, rows)
        if rows is None and self.act_dtype == torch.float32:
            post = None
            if isinstance(delta, NormedDelta):
                post, delta = delta.norm, delta.delta
            if delta is not None:
                ops.post_add_norm(x, delta, None if post is None else post.weight, 0 if post is None else post.norm_kind,
                                  0.0 if post is None else post.eps, None, ops.NORM_NONE, 0.0, None, None)
            return x
        return _post_add_norm(self, ops.NORM_COPY, x, delta, rows)
