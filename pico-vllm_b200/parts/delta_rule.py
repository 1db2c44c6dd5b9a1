"""The gated delta rule: a matrix memory per head and request whose rows decay and whose write is corrected by what the
memory already holds under the key.

With mixer input h, H heads, G query/key heads (head a reads query/key head a // (H / G)), key size d, value size d_v:

    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))      a short causal convolution per channel, as in
                                                                           :mod:`conv_attention`
    q <- q / sqrt(|q|^2 + 1e-6) * d^-1/2,   k <- k / sqrt(|k|^2 + 1e-6)    per head
    beta = sigmoid(W_b h)                                                  one per head
    a = exp( -exp(A_log) * softplus(W_a2 (W_a1 h) + dt_bias) )             one per head and row of the memory
    S <- diag(a) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q        per head, token by token
    out = W_o concat_heads( o / rms(o) * w_norm * sigmoid(W_g2 (W_g1 h)) )       w_norm [d_v], shared by the heads

State per request: S [H, d_v, d] (transposed, float32, zero at admission) and the convolution's last taps - 1 inputs.
Launches: one product for q, k, v, the beta logits and both low-rank inner vectors -> convolution (and its state) -> the two
low-rank outer products -> unit vectors, decay and beta (one kernel) -> the recurrence -> norm and gate -> output product.
Everything that enters the recurrence besides the projections and the convolution is float32, as is the memory.
The sizes of the two low-rank pairs are whatever the tensors have when the constructor is not told.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..errors import ConfigError
from .attention import _linear
from .base import FixedState, Param, Part, Piece
from .registry import register


@register("mixer", "gated_delta_rule")
class GatedDeltaRule(Part):
    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float,
                 decay_rank: Optional[int] = None, gate_rank: Optional[int] = None):
        if heads % kv_heads:
            raise ConfigError("gated_delta_rule: heads must be a multiple of kv_heads")
        if dim > 256 or not 1 <= taps <= 16:
            raise ConfigError("gated_delta_rule: a key size above 256 or a convolution beyond 16 taps is not built")
        self.width, self.heads, self.kv_heads, self.dim, self.vdim = width, heads, kv_heads, dim, vdim
        self.taps, self.eps = taps, float(eps)
        self.decay_rank, self.gate_rank = decay_rank or -1, gate_rank or -1      # -1: read from the tensor
        self.channels = 2 * kv_heads * dim + heads * vdim
        self.qkvb_weight = self.a1_weight = self.g1_weight = self.a2_weight = self.g2_weight = None
        self.proj_weight = self.conv_weight = self.dt_bias = self.a_log = self.out_norm = self.o_weight = None

    def params(self) -> List[Param]:
        qk, v, H, D = self.kv_heads * self.dim, self.heads * self.vdim, self.heads, self.width
        return [Param("qkvb_weight", (Piece("q.weight", (qk, D)), Piece("k.weight", (qk, D)), Piece("v.weight", (v, D)),
                                      Piece("b.weight", (H, D)))),
                Param("a1_weight", (Piece("a1.weight", (self.decay_rank, D)),)),
                Param("g1_weight", (Piece("g1.weight", (self.gate_rank, D)),)),
                Param("a2_weight", (Piece("a2.weight", (H * self.dim, self.decay_rank)),)),
                Param("g2_weight", (Piece("g2.weight", (v, self.gate_rank)),)),
                Param("conv_weight", (Piece("q.conv", (qk, self.taps)), Piece("k.conv", (qk, self.taps)),
                                      Piece("v.conv", (v, self.taps))), kind="vector", init="const:0.3"),
                Param("dt_bias", (Piece("dt_bias", (H * self.dim,)),), kind="vector"),
                Param("a_log", (Piece("A_log", (H,)),), kind="vector"),
                Param("out_norm", (Piece("norm", (self.vdim,)),), kind="vector", init="one_plus_normal"),
                Param("o_weight", (Piece("o.weight", (D, v)),))]

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "out_norm":
            tensor = tensor.repeat(self.heads).contiguous()      # the kernel wants a weight per column
        setattr(self, attr, tensor)

    def materialize(self, device, dtype):
        """One matrix for everything that is multiplied with h: q | k | v | beta logits | W_a1 | W_g1, each part starting at a
        multiple of 8 rows (16 bytes of a bfloat16 output row)."""
        if self.qkvb_weight is None or self.proj_weight is not None:
            return
        pad = lambda t: t if t.shape[0] % 8 == 0 else torch.cat([t, t.new_zeros((8 - t.shape[0] % 8, t.shape[1]))], 0)
        parts = [pad(self.qkvb_weight), pad(self.a1_weight), pad(self.g1_weight)]
        self.b_off = self.channels
        self.a1_off = parts[0].shape[0]
        self.g1_off = self.a1_off + parts[1].shape[0]
        self.decay_rank, self.gate_rank = self.a1_weight.shape[0], self.g1_weight.shape[0]
        if len({p.dtype for p in parts}) > 1:
            parts = [p.to(torch.float32) for p in parts]
        n0, n1, n2 = self.qkvb_weight.shape[0], self.decay_rank, self.gate_rank
        self.proj_weight = torch.cat(parts, 0).contiguous()
        # the three parameters live on as rows of the one matrix
        self.qkvb_weight = self.proj_weight[:n0]
        self.a1_weight = self.proj_weight[self.a1_off:self.a1_off + n1]
        self.g1_weight = self.proj_weight[self.g1_off:self.g1_off + n2]

    def cache_spec(self):
        return (FixedState((self.heads, self.vdim, self.dim), "float32"),
                FixedState((self.taps - 1, self.channels), "float32"))

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        H, G, d, dv = self.heads, self.kv_heads, self.dim, self.vdim
        memory, conv_state = cache
        proj = _linear(h, self.proj_weight)                      # [T, q | k | v | beta logits | a1 | g1]
        xc = ops.causal_conv_silu(proj, 0, self.conv_weight, None, conv_state.state, batch.tok_seg, batch.seg_slots,
                                  batch.cu_q, batch.positions)                               # float32 [T, q | k | v]
        dt = ops.linear(proj[:, self.a1_off:self.a1_off + self.decay_rank], self.a2_weight)  # [T, H d]
        gate = ops.linear(proj[:, self.g1_off:self.g1_off + self.gate_rank], self.g2_weight)  # [T, H dv]
        prep = ops.delta_prepare(xc, 0, G * d, proj, self.b_off, dt, self.dt_bias, self.a_log, H, G, d)
        o = ops.gated_delta_rule(prep, xc[:, 2 * G * d:], memory.state, batch.seg_slots, batch.cu_q, batch.positions,
                                 H, G, d, dv)
        y = ops.group_rms_norm(o, H, dv, dv, self.out_norm, self.eps, h.dtype, post_gate=gate)
        return _linear(y, self.o_weight)
