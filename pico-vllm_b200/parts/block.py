"""Arrangement of parts in one layer: pre-norm residual block.

x += mixer(norm1(x)); x += feed_forward(norm2(x))  (pico_vllm/model.py:361-374).  The adds are
not done here: a block hands the not-yet-added output of its feed-forward to whoever norms next
(the next block or the last norm), so that every add is fused into a norm kernel.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import CacheView, Part


class PreNormBlock:
    def __init__(self, norm1: Part, mixer: Part, norm2: Optional[Part] = None, feed_forward: Optional[Part] = None):
        """``feed_forward`` (with ``norm2``) may be None: the layer is then its mixer alone."""
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        p = {"norm1": self.norm1, "mixer": self.mixer}
        if self.feed_forward is not None:
            p.update(norm2=self.norm2, feed_forward=self.feed_forward)
        return p

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], batch,
                cache: CacheView) -> Tuple[torch.Tensor, torch.Tensor]:
        """x: float32 residual stream [T, width]; pending: output of the previous part that is
        still to be added to x (or None).  Returns (x, pending) in the same sense."""
        a = self._run(self.norm1, self.mixer, x, pending, batch, cache)
        if self.feed_forward is None:
            return x, a
        return x, self._run(self.norm2, self.feed_forward, x, a, batch)

    @staticmethod
    def _run(norm, part, x, pending, *args):
        """norm, then the part.  A part that says ``fuses_residual`` may add its output to x itself
        and return None; one that also has ``can_fuse_norm`` may take x and the norm instead of
        normed activations (when nothing is pending to be added first)."""
        fuses = getattr(part, "fuses_residual", False)
        if fuses and pending is None and hasattr(part, "can_fuse_norm") and part.can_fuse_norm(x, norm):
            return part.forward(None, *args, residual=x, norm=norm)
        h = norm.add_norm(x, pending)
        if fuses:
            return part.forward(h, *args, residual=x)
        return part.forward(h, *args)


class ParallelBlock:
    """A layer with ONE norm whose mixer and feed-forward both read its output and whose outputs are added together:
    h = norm1(x); x += mixer(h) + feed_forward(h).  ``feed_forward`` may be None.  ``side`` (optional; a part with
    ``read_norm``, ``forward(x_act, batch) -> delta`` and ``out_norm``): after that add, something made from the stream itself
    and the batch's tokens passes through ``side.out_norm`` and is added too.  The adds are not done here: the outputs travel
    on as one :class:`~pico_vllm_b200.parts.norm.SumDelta` (a mixer may hand back one of its own), the side's as a
    :class:`~pico_vllm_b200.parts.norm.NormedDelta`, so that each add happens inside the kernel of whoever reads next."""

    def __init__(self, norm1: Part, mixer: Part, feed_forward: Optional[Part] = None, side: Optional[Part] = None):
        self.norm1, self.mixer, self.feed_forward, self.side = norm1, mixer, feed_forward, side

    def parts(self):
        p = {"norm1": self.norm1, "mixer": self.mixer}
        if self.feed_forward is not None:
            p["feed_forward"] = self.feed_forward
        if self.side is not None:
            p.update(side=self.side, side_norm=self.side.out_norm)
        return p

    def forward(self, x: torch.Tensor, pending, batch, cache: CacheView):
        from .norm import NormedDelta, SumDelta
        h = self.norm1.add_norm(x, pending)
        a = self.mixer.forward(h, batch, cache)
        terms = list(a.terms) if isinstance(a, SumDelta) else [(a, None, 1.0)]
        if self.feed_forward is not None:
            terms.append((self.feed_forward.forward(h, batch), None, 1.0))
        delta = SumDelta(terms)
        if self.side is None:
            return x, delta
        xa = self.side.read_norm.add_norm(x, delta)          # the adds, and the stream in the activation type
        return x, NormedDelta(self.side.forward(xa, batch), self.side.out_norm)


class SandwichBlock:
    """A layer that norms each sublayer's input and its output:  x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))).
    ``feed_forward`` (with ``norm2`` and ``norm2b``) may be None: the layer is then its mixer alone.  A sublayer's
    output travels on as a :class:`~pico_vllm_b200.parts.norm.NormedDelta`, so that its norm, the add and the next
    sublayer's input norm are one kernel."""

    def __init__(self, norm1: Part, mixer: Part, norm1b: Part, norm2: Optional[Part] = None,
                 feed_forward: Optional[Part] = None, norm2b: Optional[Part] = None):
        self.norm1, self.mixer, self.norm1b = norm1, mixer, norm1b
        self.norm2, self.feed_forward, self.norm2b = norm2, feed_forward, norm2b

    def parts(self):
        p = {"norm1": self.norm1, "mixer": self.mixer, "norm1b": self.norm1b}
        if self.feed_forward is not None:
            p.update(norm2=self.norm2, feed_forward=self.feed_forward, norm2b=self.norm2b)
        return p

    def forward(self, x: torch.Tensor, pending, batch, cache: CacheView):
        from .norm import NormedDelta
        h = self.norm1.add_norm(x, pending)
        pending = NormedDelta(self.mixer.forward(h, batch, cache), self.norm1b)
        if self.feed_forward is None:
            return x, pending
        h = self.norm2.add_norm(x, pending)
        return x, NormedDelta(self.feed_forward.forward(h, batch), self.norm2b)
