"""Softmax attention without rotation whose positions enter as a distance bias, and two mixers side by side.

:class:`DistanceBiasAttention` - grouped-query attention over the paged cache with, each an option of its own:

    q = W_q h, k = W_k h, v = W_v h                                   (H query heads of d, G key/value heads of d and d_v)
    whole_qk_norm:  q <- q / rms(all H d numbers of q) * w_q,  k likewise over its G d numbers with w_k
    value_norm:     each head's v <- v / rms(v)  (no weight); it is cached so
    s(i, j) = scale * q_i . k_j - slope_h * (i - j),   slope_h = 2^(-8 (h + 1) / H)                     (distance_bias)
    chunk C:        position i sees j <= i only when floor(i / C) = floor(j / C), counted from the request's start
    sink:           p_j = exp(s_j) / (exp(sink) + sum_j exp(s_j)) with sink = 0: a key of score 0 that has no value
    out = W_o concat_heads(sum_j p_j v_j)

Launches: one product for q, k, v -> norms and cache store (one kernel) -> paged attention -> output product.  Norms, scores
and the softmax are float32.  Query/key size and value size may differ: heads are padded with zeros to one size in the
cache and in the kernels.

:class:`ParallelMixers` - two mixers that read the same input; the result is a_left * left + a_right * right.
"""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import ops
from .attention import AttentionPlan, _linear, decode_splits
from .base import CacheView, MixerPlan, PagedKV, Param, Part, Piece, StepShape
from .registry import register


@register("mixer", "distance_bias_attention")
class DistanceBiasAttention(Part):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, eps: float, scale: Optional[float] = None,
                 whole_qk_norm: bool = True, value_norm: bool = True, distance_bias: bool = True, chunk: Optional[int] = None,
                 sink: Optional[float] = 0.0, window: Optional[int] = None):
        self.width, self.n_heads, self.n_kv_heads, self.dim, self.vdim = width, n_heads, n_kv_heads, dim, vdim
        self.row = -(-max(dim, vdim) // 16) * 16         # a head in the cache and the kernels: padded with zeros
        self.eps, self.scale = float(eps), dim ** -0.5 if scale is None else float(scale)
        self.whole_qk_norm, self.value_norm, self.distance_bias = whole_qk_norm, value_norm, distance_bias
        self.chunk, self.sink, self.window = chunk, sink, window
        self.proj_weight = self.q_norm = self.k_norm = self.o_weight = self.slopes = self.sinks = None

    def params(self) -> List[Param]:
        q, k, v = self.n_heads * self.dim, self.n_kv_heads * self.dim, self.n_kv_heads * self.vdim
        ps = [Param("proj_weight", (Piece("q.weight", (q, self.width)), Piece("k.weight", (k, self.width)),
                                    Piece("v.weight", (v, self.width)))),
              Param("o_weight", (Piece("o.weight", (self.width, self.n_heads * self.vdim)),))]
        if self.whole_qk_norm:
            ps += [Param("q_norm", (Piece("q.norm", (q,)),), kind="vector", init="one_plus_normal"),
                   Param("k_norm", (Piece("k.norm", (k,)),), kind="vector", init="one_plus_normal")]
        return ps

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "o_weight" and self.row != self.vdim:          # the kernels hand back heads of ``row`` elements
            t = tensor.view(self.width, self.n_heads, self.vdim)
            tensor = torch.cat([t, t.new_zeros(self.width, self.n_heads, self.row - self.vdim)], 2).reshape(self.width, -1)
        setattr(self, attr, tensor.contiguous())

    def cache_spec(self):
        return PagedKV(self.n_kv_heads, self.row, self.window)

    def materialize(self, device, dtype):
        H = self.n_heads
        if self.distance_bias:
            self.slopes = torch.tensor([2.0 ** (-8.0 * (a + 1) / H) for a in range(H)], dtype=torch.float32, device=device)
        if self.sink is not None:
            self.sinks = torch.full((H,), float(self.sink), dtype=torch.float32, device=device)

    def plan_key(self):
        return ("distance_bias_attention", self.n_heads, self.n_kv_heads, self.row, self.window, self.chunk)

    def plan(self, shape: StepShape) -> AttentionPlan:
        splits = decode_splits(shape, self.n_kv_heads)
        if self.chunk:                                           # no token reads more keys than a chunk holds: parts of
            while splits > 1 and splits * 512 > self.chunk:      # 512 keys at least
                splits //= 2
        scratch = ops.attention_scratch_floats(shape.num_tokens, self.n_heads, self.row, splits)
        return AttentionPlan(key=(splits, 0), scratch_floats=scratch, splits=splits, pair_min_keys=0)

    def forward(self, h: torch.Tensor, batch, cache: CacheView) -> torch.Tensor:
        gb = batch.groups[cache.group]
        slots = gb.slots if cache.store else None
        H, G, d, dv, row = self.n_heads, self.n_kv_heads, self.dim, self.vdim, self.row
        proj = _linear(h, self.proj_weight)                      # [T, q | k | v]
        q = ops.whole_norm_store(proj, 0, H * d, (H + G) * d, self.q_norm, self.k_norm, self.eps, self.value_norm, slots,
                                 cache.k, cache.v, H, G, d, dv, row, cache.page_size)
        out = torch.empty((h.shape[0], H * row), dtype=h.dtype, device=h.device)
        plan = batch.plan(self)
        splits = plan.splits if plan is not None else 1
        if ops.mma_attention_takes(h.dtype, H, G, row):
            ops.paged_attention_mma(q, cache.k, cache.v, out, batch.tok_seg, batch.positions, gb.block_table, batch.cu_q,
                                    batch.prefill_segs, batch.num_prefill_segs, batch.max_prefill_q, batch.decode_tokens,
                                    batch.num_decode_tokens, H, G, row, cache.page_size, self.window, self.scale, splits,
                                    batch.scratch, None, None, cache.k_map2d, cache.v_map2d, 0, slopes=self.slopes,
                                    chunk=self.chunk, sinks=self.sinks)
        else:       # float32, or sizes the tensor-core kernels do not take
            ops.paged_attention(q, cache.k, cache.v, out, batch.tok_seg, batch.positions, gb.block_table, H, G, row,
                                cache.page_size, self.window, self.scale, splits, batch.scratch, slopes=self.slopes,
                                chunk=self.chunk, sinks=self.sinks)
        return _linear(out, self.o_weight)


@register("mixer", "parallel_mixers")
class ParallelMixers(Part):
    """Two mixers on the same input, left_scale * left(h) + right_scale * right(h).  Tensor keys of the two are prefixed
    ``left.`` and ``right.``; each keeps its own cache entries."""

    def __init__(self, left: Part, right: Part, left_scale: float = 1.0, right_scale: float = 1.0,
                 left_norm: Optional[Part] = None, right_norm: Optional[Part] = None):
        """``left_norm`` / ``right_norm`` (RMS norms over the model width, tensor keys ``left.out`` / ``right.out``): each
        side's output passes through its norm before the scaled sum; the mixer then hands back a
        :class:`~pico_vllm_b200.parts.norm.SumDelta` and the sum happens where the residual stream is next touched."""
        self.left, self.right, self.left_scale, self.right_scale = left, right, float(left_scale), float(right_scale)
        self.left_norm, self.right_norm = left_norm, right_norm
        self._n_left = len(_as_tuple(left.cache_spec()))

    def _sides(self):
        return (("left", self.left), ("right", self.right))

    def params(self) -> List[Param]:
        out = []
        for name, part in self._sides():
            for p in part.params():
                out.append(Param(f"{name}__{p.attr}", tuple(Piece(f"{name}.{pc.key}", pc.shape) for pc in p.pieces),
                                 kind=p.kind, init=p.init))
        for name, norm in (("left", self.left_norm), ("right", self.right_norm)):
            if norm is not None:
                for p in norm.params():
                    out.append(Param(f"{name}norm__{p.attr}", tuple(Piece(f"{name}.out", pc.shape) for pc in p.pieces),
                                     kind=p.kind, init=p.init))
        return out

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        side, _, inner = attr.partition("__")
        if side in ("leftnorm", "rightnorm"):
            getattr(self, side[:-4] + "_norm").assign(inner, tensor)
            return
        getattr(self, side).assign(inner, tensor)

    def __getattr__(self, attr: str):
        """A parameter of one side under the name ``params`` gives it (``left__proj_weight``)."""
        side, sep, inner = attr.partition("__")
        if sep and side in ("left", "right") and inner:
            return getattr(self.__dict__[side], inner)
        if sep and side in ("leftnorm", "rightnorm") and inner:
            return getattr(self.__dict__[side[:-4] + "_norm"], inner)
        raise AttributeError(attr)

    def cache_spec(self):
        return _as_tuple(self.left.cache_spec()) + _as_tuple(self.right.cache_spec())

    def materialize(self, device, dtype):
        self.left.materialize(device, dtype)
        self.right.materialize(device, dtype)
        for norm in (self.left_norm, self.right_norm):
            if norm is not None:
                norm.materialize(device, dtype)

    def plan_key(self):
        return ("parallel_mixers", self.left.plan_key(), self.right.plan_key())

    def plan(self, shape: StepShape):
        """The plans of both sides under one key; each side finds its own through ``batch.plan``."""
        lp, rp = self.left.plan(shape), self.right.plan(shape)
        if lp is None and rp is None:
            return None
        return PairPlan(key=(None if lp is None else lp.key, None if rp is None else rp.key),
                        scratch_floats=max(0 if lp is None else lp.scratch_floats, 0 if rp is None else rp.scratch_floats),
                        left=lp, right=rp)

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        views = _as_tuple(cache)
        lv, rv = views[:self._n_left], views[self._n_left:]
        own = batch.plan(self)
        with _side_plan(batch, self.left, None if own is None else own.left):
            a = self.left.forward(h, batch, lv[0] if len(lv) == 1 else lv)
        with _side_plan(batch, self.right, None if own is None else own.right):
            b = self.right.forward(h, batch, rv[0] if len(rv) == 1 else rv)
        if self.left_norm is not None or self.right_norm is not None:
            from .norm import SumDelta
            return SumDelta([(a, self.left_norm, self.left_scale), (b, self.right_norm, self.right_scale)])
        return ops.scaled_sum(a, self.left_scale, b, self.right_scale)


def _as_tuple(x):
    if x is None:
        return ()
    return tuple(x) if isinstance(x, (tuple, list)) else (x,)


@dataclass(frozen=True)
class PairPlan(MixerPlan):
    left: object = None
    right: object = None


@contextmanager
def _side_plan(batch, part, plan):
    """While one side runs, its plan stands in the batch under the side's own key."""
    key = part.plan_key()
    had, old = key in batch.plans, batch.plans.get(key)
    if plan is not None:
        batch.plans[key] = plan
    try:
        yield
    finally:
        if plan is not None:
            if had:
                batch.plans[key] = old
            else:
                del batch.plans[key]
