"""Grouped-query softmax attention whose projections pass a short causal convolution, with neighbouring dimensions rotated
together and queries and keys normed after the rotation.

With mixer input h, H query heads, G key/value heads (query head a reads key/value head a // (H / G)), query/key size d,
value size d_v, ``taps`` convolution taps:

    q, k, v = conv(W_q h), conv(W_k h), conv(W_v h)       conv(u)_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the
                                                          request's start, one weight row per channel, no activation
    q, k:  (x[2i], x[2i+1]) <- (x[2i] cos a - x[2i+1] sin a, x[2i+1] cos a + x[2i] sin a),  a = position * base^(-2i / rot_dim),
           for 2i < rot_dim; then x <- x / sqrt(mean(x^2) + eps) per head (``qk_norm``; no weight)
    out = W_o concat_heads( softmax_j<=i( scale * q_i . k_j ) v_j )

Cache: keys and values in pages (heads padded with zeros to one size when d and d_v differ), and the last taps - 1
projected rows of the request in a state slot, so that a portion goes on where the one before stopped.
Launches: one product for q, k, v -> convolution (and its state) -> rotation, norm and cache store (one kernel) -> paged
attention -> output product.  Convolution, angles, rotation, norm, scores and softmax are float32.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .attention import AttentionPlan, _linear, decode_splits
from .base import FixedState, PagedKV, Param, Part, Piece, StepShape
from .registry import register


@register("mixer", "conv_rope_attention")
class ConvRopeAttention(Part):
    def __init__(self, width: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, eps: float, scale: Optional[float] = None,
                 taps: int = 1, rot_base: Optional[float] = None, rot_dim: int = 0, qk_norm: bool = True,
                 window: Optional[int] = None):
        self.width, self.n_heads, self.n_kv_heads, self.dim, self.vdim = width, n_heads, n_kv_heads, dim, vdim
        self.row = -(-max(dim, vdim) // 16) * 16         # a head in the cache and the kernels: padded with zeros
        self.eps, self.scale = float(eps), dim ** -0.5 if scale is None else float(scale)
        self.taps, self.rot_base, self.rot_dim = taps, rot_base, (rot_dim if rot_base else 0)
        self.qk_norm, self.window = qk_norm, window
        self.channels = (n_heads + n_kv_heads) * dim + n_kv_heads * vdim
        self.proj_weight = self.conv_weight = self.o_weight = self.inv_freq = None

    def params(self) -> List[Param]:
        q, k, v = self.n_heads * self.dim, self.n_kv_heads * self.dim, self.n_kv_heads * self.vdim
        return [Param("proj_weight", (Piece("q.weight", (q, self.width)), Piece("k.weight", (k, self.width)),
                                      Piece("v.weight", (v, self.width)))),
                Param("conv_weight", (Piece("q.conv", (q, self.taps)), Piece("k.conv", (k, self.taps)),
                                      Piece("v.conv", (v, self.taps))), kind="vector", init="const:0.3"),
                Param("o_weight", (Piece("o.weight", (self.width, self.n_heads * self.vdim)),))]

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "o_weight" and self.row != self.vdim:          # the kernels hand back heads of ``row`` elements
            t = tensor.view(self.width, self.n_heads, self.vdim)
            tensor = torch.cat([t, t.new_zeros(self.width, self.n_heads, self.row - self.vdim)], 2).reshape(self.width, -1)
        setattr(self, attr, tensor.contiguous())

    def cache_spec(self):
        return (PagedKV(self.n_kv_heads, self.row, self.window), FixedState((self.taps - 1, self.channels), "float32"))

    def materialize(self, device, dtype):
        if self.rot_dim:
            i = torch.arange(self.rot_dim // 2, dtype=torch.float64)
            self.inv_freq = (float(self.rot_base) ** (-2.0 * i / self.rot_dim)).to(torch.float32).to(device)

    def plan_key(self):
        return ("conv_rope_attention", self.n_heads, self.n_kv_heads, self.row, self.window)

    def plan(self, shape: StepShape) -> AttentionPlan:
        splits = decode_splits(shape, self.n_kv_heads)
        scratch = ops.attention_scratch_floats(shape.num_tokens, self.n_heads, self.row, splits)
        return AttentionPlan(key=(splits, 0), scratch_floats=scratch, splits=splits, pair_min_keys=0)

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        pages, conv_state = cache
        gb = batch.groups[pages.group]
        slots = gb.slots if pages.store else None
        H, G, d, dv, row = self.n_heads, self.n_kv_heads, self.dim, self.vdim, self.row
        proj = _linear(h, self.proj_weight)                      # [T, q | k | v]
        xc = ops.causal_conv_silu(proj, 0, self.conv_weight, None, conv_state.state, batch.tok_seg, batch.seg_slots,
                                  batch.cu_q, batch.positions, act=False)                    # float32 [T, q | k | v]
        q = ops.pair_rope_norm_store(xc, 0, H * d, (H + G) * d, batch.positions, self.inv_freq, self.qk_norm, None, None,
                                     self.eps, slots, pages.k, pages.v, H, G, d, dv, row, pages.page_size, h.dtype)
        out = torch.empty((h.shape[0], H * row), dtype=h.dtype, device=h.device)
        plan = batch.plan(self)
        splits = plan.splits if plan is not None else 1
        if ops.mma_attention_takes(h.dtype, H, G, row):
            ops.paged_attention_mma(q, pages.k, pages.v, out, batch.tok_seg, batch.positions, gb.block_table, batch.cu_q,
                                    batch.prefill_segs, batch.num_prefill_segs, batch.max_prefill_q, batch.decode_tokens,
                                    batch.num_decode_tokens, H, G, row, pages.page_size, self.window, self.scale, splits,
                                    batch.scratch, pages.k_map, pages.v_map, pages.k_map2d, pages.v_map2d, 0)
        else:       # float32, or sizes the tensor-core kernels do not take
            ops.paged_attention(q, pages.k, pages.v, out, batch.tok_seg, batch.positions, gb.block_table, H, G, row,
                                pages.page_size, self.window, self.scale, splits, batch.scratch)
        return _linear(out, self.o_weight)
