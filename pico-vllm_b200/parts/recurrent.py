"""Mixers whose memory is a matrix of fixed size per request, with gates that depend on the token.

All three are the recurrence  S_t = diag(a_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t  per head (one kernel,
``ops.gated_linear_attention``) behind different gates, between one product for all projections and one norm kernel that
finishes the heads' outputs (``ops.group_rms_norm``) before the output product.  The state lives in float32 in fixed-size
slots of the cache manager (zeroed when a request is admitted) and is carried from step to step: a portion of a prompt goes
on where the one before stopped, a decoded token is a portion of one.  Gates, step sizes, decays, the recurrence and the
norms are float32 whatever the activation type.

* :class:`ExpGatedMatrixMemory` - the matrix memory of xLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory"): an
  input gate and a forget gate per head that live as logarithms, kept finite by a running maximum, and a normaliser.
* :class:`ForgetWriteLinearAttention` - HGRN2 (Qin et al., "HGRN2: Gated Linear RNNs with State Expansion"): the forget
  gate per row of the state also decides what is written (the key is 1 - f).
* :class:`StateSpaceDuality` - Mamba-2 (Dao and Gu, "Transformers are SSMs"): a short causal convolution, a step size and a
  decay per head, a skip term, a gate before a grouped norm.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..errors import ConfigError
from .attention import _linear
from .base import FixedState, Param, Part, Piece
from .registry import register


def _max_q(batch) -> int:
    return max(batch.q_lens, default=1)


@register("mixer", "exp_gated_matrix_memory")
class ExpGatedMatrixMemory(Part):
    """With mixer input h, H heads, key size d, value size d_v and the cap c on the gates' arguments:

        q = W_q h / sqrt(d),  k = W_k h,  v = W_v h
        i = c tanh((W_i h + b_i) / c),   f = logsigmoid(c tanh((W_f h + b_f) / c))          (one of each per head)
        m_t = max(f + m_(t-1), i)                                                            (m_0 = 0)
        S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T ,   n_t the same with k alone
        o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
        out = W_o ( concat_heads(o / rms(o)) * w_norm * sigmoid(W_g h) )

    State per request: S with n as one more column [H, d_v + 1, d] (transposed), and m [H]."""

    def __init__(self, width: int, heads: int, dim: int, vdim: int, gate_cap: float, eps: float):
        if dim > 256:
            raise ConfigError(f"exp_gated_matrix_memory: key size {dim} above 256 is not built")
        if not gate_cap > 0:
            raise ConfigError("exp_gated_matrix_memory: the gate cap must be positive")
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        self.proj_weight = self.gate_bias = self.out_norm = self.o_weight = None

    def params(self) -> List[Param]:
        qk, v, H, D = self.heads * self.dim, self.heads * self.vdim, self.heads, self.width
        return [Param("proj_weight", (Piece("q.weight", (qk, D)), Piece("k.weight", (qk, D)), Piece("v.weight", (v, D)),
                                      Piece("g.weight", (v, D)), Piece("i.weight", (H, D)), Piece("f.weight", (H, D)))),
                Param("gate_bias", (Piece("i.bias", (H,)), Piece("f.bias", (H,))), kind="vector"),
                Param("out_norm", (Piece("norm", (v,)),), kind="vector", init="one_plus_normal"),
                Param("o_weight", (Piece("o.weight", (D, v)),))]

    def cache_spec(self):
        return (FixedState((self.heads, self.vdim + 1, self.dim), "float32"), FixedState((self.heads,), "float32"))

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        H, d, dv = self.heads, self.dim, self.vdim
        memory, running_max = cache
        proj = _linear(h, self.proj_weight)                      # [T, q | k | v | gate logits | i | f]
        v0, g0 = 2 * H * d, 2 * H * d + H * dv
        i0 = g0 + H * dv
        keep, floor, prep = ops.mlstm_prepare(proj, 0, H * d, v0, i0, i0 + H, self.gate_bias[:H], self.gate_bias[H:],
                                              self.gate_cap, d ** -0.5, running_max.state, batch.seg_slots, batch.cu_q,
                                              batch.positions, H, d, dv)
        o = ops.gated_linear_attention(prep[:, :H * d], prep[:, H * d:v0], prep[:, v0:], keep, False, memory.state,
                                       batch.seg_slots, batch.cu_q, batch.positions, H, 1, d, dv + 1, max_q_len=_max_q(batch))
        y = ops.group_rms_norm(o, H, dv, dv + 1, self.out_norm, self.eps, h.dtype, den_floor=floor,
                               post_gate=proj[:, g0:g0 + H * dv])
        return _linear(y, self.o_weight)


@register("mixer", "forget_write_linear_attention")
class ForgetWriteLinearAttention(Part):
    """With H heads, query size d and value size d_v:

        q = silu(W_q h),  v = W_v h,  f = l + (1 - l) sigmoid(W_f h + b_f)        (f, and the lower bound l, per head and row)
        S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T ,   o_t = S_t^T q_t
        out = W_o concat_heads( o / rms(o) * w_norm )                              (w_norm [d_v], shared by the heads)

    State per request: S [H, d_v, d] (transposed)."""

    def __init__(self, width: int, heads: int, dim: int, vdim: int, eps: float):
        if dim > 256:
            raise ConfigError(f"forget_write_linear_attention: query size {dim} above 256 is not built")
        self.width, self.heads, self.dim, self.vdim, self.eps = width, heads, dim, vdim, float(eps)
        self.proj_weight = self.f_bias = self.lower = self.out_norm = self.o_weight = None

    def params(self) -> List[Param]:
        qk, v, D = self.heads * self.dim, self.heads * self.vdim, self.width
        return [Param("proj_weight", (Piece("q.weight", (qk, D)), Piece("f.weight", (qk, D)), Piece("v.weight", (v, D)))),
                Param("f_bias", (Piece("f.bias", (qk,)),), kind="vector"),
                Param("lower", (Piece("lower", (qk,)),), kind="vector", init="const:0.3"),
                Param("out_norm", (Piece("norm", (self.vdim,)),), kind="vector", init="one_plus_normal"),
                Param("o_weight", (Piece("o.weight", (D, v)),))]

    def assign(self, attr: str, tensor: torch.Tensor) -> None:
        if attr == "out_norm":
            tensor = tensor.repeat(self.heads).contiguous()      # the kernel wants a weight per column
        setattr(self, attr, tensor)

    def cache_spec(self):
        return FixedState((self.heads, self.vdim, self.dim), "float32")

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        H, d, dv = self.heads, self.dim, self.vdim
        n = H * d
        proj = _linear(h, self.proj_weight)                      # [T, q | f | v]
        prep = ops.hgrn2_prepare(proj, 0, n, 2 * n, self.f_bias, self.lower, n, H * dv)      # [T, q | k | f | v]
        o = ops.gated_linear_attention(prep[:, :n], prep[:, n:2 * n], prep[:, 3 * n:], prep[:, 2 * n:3 * n], True, cache.state,
                                       batch.seg_slots, batch.cu_q, batch.positions, H, 1, d, dv, max_q_len=_max_q(batch))
        y = ops.group_rms_norm(o, H, dv, dv, self.out_norm, self.eps, h.dtype)
        return _linear(y, self.o_weight)


@register("mixer", "state_space_duality")
class StateSpaceDuality(Part):
    """With H heads of size P, state size N, G groups of B and C (head h uses group h // (H / G)), inner = H P:

        W_in h = [z: inner | x: inner | B: G N | C: G N | dt: H];   x, B, C <- silu(causal convolution per channel, ``taps`` long)
        dt <- softplus(dt + dt_bias);   S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T ;   y_t = S_t^T C_t + D x_t
        out = W_o ( rms in ``norm_groups`` equal parts of (y * silu(z)) * w_norm )

    State per request: S [H, P, N] (transposed) and the last taps - 1 inputs of the convolution [taps - 1, inner + 2 G N]."""

    def __init__(self, width: int, heads: int, vdim: int, state: int, groups: int, conv: int, norm_groups: int, eps: float):
        if heads % groups or (heads * vdim) % norm_groups:
            raise ConfigError("state_space_duality: heads must be a multiple of groups, heads * vdim of norm_groups")
        if state > 256 or not 1 <= conv <= 16:
            raise ConfigError("state_space_duality: a state above 256 or a convolution beyond 16 taps is not built")
        self.width, self.heads, self.vdim, self.state, self.groups = width, heads, vdim, state, groups
        self.taps, self.norm_groups, self.eps = conv, norm_groups, float(eps)
        self.inner = heads * vdim
        self.channels = self.inner + 2 * groups * state
        self.in_weight = self.conv_weight = self.conv_bias = self.dt_bias = self.a_log = self.skip = None
        self.out_norm = self.o_weight = None

    def params(self) -> List[Param]:
        H, D, C = self.heads, self.width, self.channels
        return [Param("in_weight", (Piece("in.weight", (self.inner + C + H, D)),)),
                Param("conv_weight", (Piece("conv.weight", (C, self.taps)),), kind="vector", init="const:0.25"),
                Param("conv_bias", (Piece("conv.bias", (C,)),), kind="vector"),
                Param("dt_bias", (Piece("dt_bias", (H,)),), kind="vector"),
                Param("a_log", (Piece("A_log", (H,)),), kind="vector"),
                Param("skip", (Piece("D", (H,)),), kind="vector", init="one_plus_normal"),
                Param("out_norm", (Piece("norm", (self.inner,)),), kind="vector", init="one_plus_normal"),
                Param("o_weight", (Piece("o.weight", (D, self.inner)),))]

    def cache_spec(self):
        return (FixedState((self.heads, self.vdim, self.state), "float32"),
                FixedState((self.taps - 1, self.channels), "float32"))

    def forward(self, h: torch.Tensor, batch, cache) -> torch.Tensor:
        H, P, N, G, inner = self.heads, self.vdim, self.state, self.groups, self.inner
        memory, conv_state = cache
        proj = _linear(h, self.in_weight)                        # [T, z | x | B | C | dt]
        xbc = ops.causal_conv_silu(proj, inner, self.conv_weight, self.conv_bias, conv_state.state, batch.tok_seg,
                                   batch.seg_slots, batch.cu_q, batch.positions)             # float32 [T, x | B | C]
        keep, vdt = ops.mamba2_prepare(proj, inner + self.channels, self.dt_bias, self.a_log, xbc[:, :inner], H, P)
        o = ops.gated_linear_attention(xbc[:, inner + G * N:], xbc[:, inner:inner + G * N], vdt, keep, False, memory.state,
                                       batch.seg_slots, batch.cu_q, batch.positions, H, H // G, N, P, max_q_len=_max_q(batch))
        part = inner // self.norm_groups
        y = ops.group_rms_norm(o, self.norm_groups, part, part, self.out_norm, self.eps, h.dtype, skip=xbc[:, :inner],
                               skip_w=self.skip, skip_head=P, pre_gate=proj[:, :inner])
        return _linear(y, self.o_weight)
