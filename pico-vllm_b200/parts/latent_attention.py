"""Latent attention: keys and values of all heads are made from one small cached vector per token.

For a token with mixer input h (width D), H heads, query/key size d, value size d_v, query latent rank r_q and
cached latent rank r:

    c_q = rms(W_dq h) * w_q                   (r_q)         c = rms(W_dkv h) * w_kv      (r; the only thing cached)
    q_a = W_uq[a] c_q                         (d)           k_a(j) = W_uk[a] c(j),  v_a(j) = W_uv[a] c(j)
    p_a(j) = softmax_j( scale * q_a . k_a(j) )  over the visible positions j <= i
    out = W_o concat_a( sigmoid(W_g h)_a * sum_j p_a(j) v_a(j) )

No position encoding acts on q or k.  A layer may read the latents another layer caches (``own_latent=False``: it
has no W_dkv; its cache entry is that layer's).  Options: ``q_rank=None`` - the queries are projected directly, q = W_q h
(no query latent, no norm on that side); ``gate=False`` - no output gate; ``window`` W - position i sees the last W
positions, itself included.

The kernels never expand k or v.  Since q_a . (W_uk[a] c) = (W_uk[a]^T q_a) . c, the query is carried into the
latent space, q'_a = W_uk[a]^T q_a (r), attention runs over the cached latents as over ONE shared key/value head
of size r with H query heads - the paged attention kernels of this package, with the cache page tensor given as
keys and as values - and the result o'_a = sum_j p_a(j) c(j) is carried back by W_uv[a].  Prompt portions and
single tokens take the same path, so a position's logits do not depend on how its prompt was cut.

Launches of a call: down product (W_dq, W_dkv, W_g as one matrix) -> norms, cache store and gate (one kernel) ->
W_uq product -> per-head product into the latent space -> paged attention -> per-head product back -> gate ->
W_o product.  Norms, gate and softmax are float32.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .attention import AttentionPlan, decode_splits
from .base import CacheView, PagedLatent, Param, Part, Piece, StepShape
from .registry import register


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def _linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """A handful of tokens: the weight-streaming kernel; more: the library product."""
    if ops.skinny_takes(x, weight):
        return ops.skinny_linear(x, weight)
    return ops.linear(x, weight)


@register("mixer", "latent_attention")
class LatentAttention(Part):
    def __init__(self, width: int, heads: int, dim: int, vdim: int, q_rank: Optional[int], kv_rank: int, scale: float, eps: float,
                 own_latent: bool = True, window: Optional[int] = None, gate: bool = True, cache_window="same"):
        """``cache_window``: how many of the last latents the cache has to keep (None: all); by default the mixer's own
        window.  Layers that read one cache entry through different windows all name the longest."""
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.q_rank, self.kv_rank, self.scale, self.eps = q_rank, kv_rank, float(scale), float(eps)
        self.own_latent, self.window, self.gate = own_latent, window, gate
        self.cache_window = window if cache_window == "same" else cache_window
        self.row = _round_up(kv_rank, 16)          # elements of a cache row: the attention kernels take multiples of 16
        self.down_weight = self.q_norm = self.kv_norm = self.uq_weight = self.uk_weight = self.uv_weight = None
        self.o_weight = None

    def params(self) -> List[Param]:
        down = [Piece("dq.weight", (self.q_rank, self.width))] if self.q_rank else []
        if self.own_latent:
            down.append(Piece("dkv.weight", (self.kv_rank, self.width)))
        if self.gate:
            down.append(Piece("g.weight", (self.heads, self.width)))
        ps = [Param("down_weight", tuple(down))] if down else []
        if self.q_rank:
            ps += [Param("q_norm", (Piece("dq.norm", (self.q_rank,)),), kind="vector", init="one_plus_normal"),
                   Param("uq_weight", (Piece("uq.weight", (self.heads * self.dim, self.q_rank)),))]
        else:
            ps.append(Param("uq_weight", (Piece("q.weight", (self.heads * self.dim, self.width)),)))
        ps += [Param("uk_weight", (Piece("uk.weight", (self.heads * self.dim, self.kv_rank)),)),
               Param("uv_weight", (Piece("uv.weight", (self.heads * self.vdim, self.kv_rank)),)),
               Param("o_weight", (Piece("o.weight", (self.width, self.heads * self.vdim)),))]
        if self.own_latent:
            ps.append(Param("kv_norm", (Piece("dkv.norm", (self.kv_rank,)),), kind="vector", init="one_plus_normal"))
        return ps

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        """Lays the tensors out for the kernels: the down matrix padded to a multiple of 16 rows; W_uk as
        [H, d, row] and W_uv transposed as [H, row, d_v], both with zeros beyond kv_rank."""
        pad = self.row - self.kv_rank
        if attr == "down_weight":
            extra = _round_up(tensor.shape[0], 16) - tensor.shape[0]
            if extra:
                tensor = torch.cat([tensor, tensor.new_zeros((extra, tensor.shape[1]))], 0)
        elif attr == "uk_weight":
            tensor = tensor.view(self.heads, self.dim, self.kv_rank)
            if pad:
                tensor = torch.cat([tensor, tensor.new_zeros((self.heads, self.dim, pad))], 2)
        elif attr == "uv_weight":
            tensor = tensor.view(self.heads, self.vdim, self.kv_rank).transpose(1, 2)
            if pad:
                tensor = torch.cat([tensor, tensor.new_zeros((self.heads, pad, self.vdim))], 1)
        setattr(self, attr, tensor.contiguous())

    def cache_spec(self):
        return PagedLatent(self.row, self.cache_window)

    # ------------------------------------------------------------------ launch policy of the attention kernels
    def plan_key(self):
        return ("latent_attention", self.heads, self.row, self.window)

    def plan(self, shape: StepShape) -> AttentionPlan:
        splits = decode_splits(shape, 1)
        scratch = ops.attention_scratch_floats(shape.num_tokens, self.heads, self.row, splits)
        return AttentionPlan(key=(splits, 0), scratch_floats=scratch, splits=splits, pair_min_keys=0)

    def forward(self, h: torch.Tensor, batch, cache: CacheView) -> torch.Tensor:
        """h [T, width] in the activation type; returns what is to be added to the residual stream."""
        gb = batch.groups[cache.group]
        T, H, R = h.shape[0], self.heads, self.row
        latent = cache.tensors["latent"]                       # [pages, 1, page_size, R]
        stores = self.own_latent and cache.store
        q_rank = self.q_rank or 0
        cq, gate = h, None
        if self.down_weight is not None:
            proj = _linear(h, self.down_weight)
            kv_off = q_rank
            g_off = q_rank + (self.kv_rank if self.own_latent else 0)
            cq, gate = ops.latent_norm_store(proj, 0, q_rank, self.q_norm, kv_off, self.kv_rank if stores else 0,
                                             self.kv_norm if stores else None, gb.slots if stores else None,
                                             latent if stores else None, g_off, H if self.gate else 0, self.eps)
            if not q_rank:
                cq = h
        q = _linear(cq, self.uq_weight)                         # [T, H d]: from the query latent, or from h itself
        qa = torch.empty((T, H * R), dtype=h.dtype, device=h.device)
        ops.head_linear(q, self.uk_weight, qa)                  # q'_a = W_uk[a]^T q_a
        oa = torch.empty((T, H * R), dtype=h.dtype, device=h.device)
        plan = batch.plan(self)
        splits = plan.splits if plan is not None else 1
        if ops.mma_attention_takes(h.dtype, H, 1, R):
            ops.paged_attention_mma(qa, latent, latent, oa, batch.tok_seg, batch.positions, gb.block_table, batch.cu_q,
                                    batch.prefill_segs, batch.num_prefill_segs, batch.max_prefill_q, batch.decode_tokens,
                                    batch.num_decode_tokens, H, 1, R, cache.page_size, self.window, self.scale, splits,
                                    batch.scratch, cache.k_map, cache.v_map, cache.k_map2d, cache.v_map2d, 0)
        else:       # float32, or sizes the tensor-core kernels do not take
            ops.paged_attention(qa, latent, latent, oa, batch.tok_seg, batch.positions, gb.block_table, H, 1, R,
                                cache.page_size, self.window, self.scale, splits, batch.scratch)
        o = torch.empty((T, H * self.vdim), dtype=h.dtype, device=h.device)
        ops.head_linear(oa, self.uv_weight, o, gate)            # o_a = gate_a * W_uv[a] o'_a
        return _linear(o, self.o_weight)
