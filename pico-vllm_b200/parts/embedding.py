"""Token embedding and output head.

x = E[ids] (pico_vllm/model.py:405,427) into the float32 residual stream; logits = y . W^T with
W the embedding matrix when tied (pico_vllm/model.py:445) or a matrix of its own (the reference
creates lm_head for the untied case but never uses it, pico_vllm/model.py:409-412; its older
model does, pico_vllm/legacy/model.py:223-226).  Logits are float32 and are computed only for
the rows that were asked for.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Param, Part, Piece


class TokenEmbedding(Part):
    def __init__(self, vocab: int, width: int, scale: float = 1.0):
        """``scale``: x = scale * E[ids], the product taken in float32 on the stream."""
        self.vocab, self.width, self.scale = vocab, width, float(scale)
        self.weight = None

    def params(self) -> List[Param]:
        return [Param("weight", (Piece("weight", (self.vocab, self.width)),))]

    def forward(self, ids: torch.Tensor, feedback: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = torch.empty((ids.shape[0], self.width), dtype=torch.float32, device=ids.device)
        ops.embedding(ids, self.weight, out, feedback)
        return out if self.scale == 1.0 else ops.scale_add_rows(out, self.scale, None, None)


class TokenSideTable(Part):
    """A second embedding table whose row of a token is cut into one slice per layer (``parts`` slices of ``dim``)."""

    def __init__(self, vocab: int, parts: int, dim: int):
        self.vocab, self.parts_n, self.dim = vocab, parts, dim
        self.weight = None

    def params(self) -> List[Param]:
        return [Param("weight", (Piece("weight", (self.vocab, self.parts_n * self.dim)),))]


class TokenSideInput(Part):
    """What a layer takes from the token itself, given the residual stream x (in the activation type) after the layer's
    sublayers:  g = gelu_tanh(W_gate x) * e,  y = W_proj g,  with e slice ``index`` of the token's row of ``table``; y then
    passes through ``out_norm`` (an RMS norm) on its way into the stream.  ``read_norm`` is how the block reads the stream
    for this part: no norm, the pending adds done."""

    def __init__(self, width: int, dim: int, index: int, table: TokenSideTable, out_norm: Part, read_norm: Part):
        self.width, self.dim, self.index, self.table = width, dim, index, table
        self.out_norm, self.read_norm = out_norm, read_norm
        self.gate_weight = self.proj_weight = None

    def params(self) -> List[Param]:
        return [Param("gate_weight", (Piece("gate.weight", (self.dim, self.width)),)),
                Param("proj_weight", (Piece("proj.weight", (self.width, self.dim)),))]

    def materialize(self, device, dtype):
        self.read_norm.materialize(device, dtype)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        z = ops.linear(x, self.gate_weight)
        g = ops.gelu_gate_rows(z, self.table.weight, self.index * self.dim, batch.token_ids, batch.feedback)
        return ops.linear(g, self.proj_weight)


class LearnedPositions(Part):
    """A learned vector per position, added to the residual stream right after the embedding:  x <- x * input_scale +
    table[position]  (the scale acts on the token embedding only).  A request cannot grow beyond the table."""

    def __init__(self, max_positions: int, width: int, input_scale: float = 1.0):
        self.max_positions, self.width, self.input_scale = max_positions, width, float(input_scale)
        self.weight = None

    def params(self) -> List[Param]:
        return [Param("weight", (Piece("weight", (self.max_positions, self.width)),))]

    def add_to(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        return ops.scale_add_rows(x, self.input_scale, self.weight, positions)


class OutputHead(Part):
    def __init__(self, vocab: int, width: int, tied_to: Optional[TokenEmbedding] = None, logit_scale: float = 1.0,
                 softcap: Optional[float] = None):
        """``logit_scale`` and ``softcap``: logits = softcap * tanh(logit_scale * (y . W^T) / softcap) (no cap
        when ``softcap`` is None), float32, in one kernel after the product."""
        self.vocab, self.width, self.tied_to = vocab, width, tied_to
        self.logit_scale, self.softcap = float(logit_scale), softcap
        self.weight = None

    def params(self) -> List[Param]:
        if self.tied_to is not None:
            return []
        return [Param("weight", (Piece("weight", (self.vocab, self.width)),))]

    def matrix(self) -> torch.Tensor:
        return self.tied_to.weight if self.tied_to is not None else self.weight

    def _shape(self, logits: torch.Tensor) -> torch.Tensor:
        if self.logit_scale != 1.0 or self.softcap:
            ops.scale_softcap(logits, self.logit_scale, self.softcap)
        return logits

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        return self._shape(ops.logits_linear(y, self.matrix()))

    def can_fuse_norm(self, x: torch.Tensor, norm, n_rows: int) -> bool:
        return getattr(norm, "plain_rms", False) and getattr(norm, "weight", None) is not None \
            and ops.skinny_norm_takes(x, self.matrix(), n_rows)

    def forward_normed(self, x: torch.Tensor, norm, rows: torch.Tensor) -> torch.Tensor:
        """Logits of rows ``rows`` of the residual stream x, with the last norm applied inside the kernel."""
        return self._shape(ops.skinny_linear(x, self.matrix(), None, torch.float32, norm.weight, norm.eps, rows))

    def greedy(self, x: torch.Tensor, norm, rows: Optional[torch.Tensor], n_rows: int, out: torch.Tensor) -> bool:
        """The greedy tokens of ``n_rows`` rows straight into ``out`` (int32), without logits: argmax in the
        product's epilogue.  With ``norm``, x is the residual stream and the last norm runs inside the kernel
        (``rows`` picks its rows); without, x is already normed.  False when the fused kernel does not take
        the sizes: the caller then computes logits."""
        w = self.matrix()
        if not self.logit_scale > 0.0:      # a positive scale and the cap keep the order of the logits; anything else does not
            return False
        if norm is not None:
            if not self.can_fuse_norm(x, norm, n_rows):
                return False
            ops.skinny_argmax(x, w, out, norm.weight, norm.eps, rows)
            return True
        if not ops.skinny_takes(x, w):
            return False
        ops.skinny_argmax(x, w, out)
        return True
