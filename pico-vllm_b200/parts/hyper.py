"""Several residual streams per token (hyper-connections).

Instead of one residual vector a token carries S of them, x_1 .. x_S (float32, [T, S, width]), all equal to the embedding
stage's output at the start.  A sublayer reads one mixture of them and writes to all of them:

    u = sum_s in[s] x_s ;   y = sublayer(norm(u)) ;   x_t <- sum_s mix[s, t] x_s + out[t] * y     (every t from the old x)

``in`` [S], ``out`` [S] and ``mix`` [S, S] (indexed [from, to]) are learned, per sublayer (:class:`HyperConnection`).  What
leaves the stack is the plain sum of the streams.  The write of one sublayer and the read (with its norm) of the next are
one kernel: a sublayer's output travels on as a :class:`HyperDelta` until the next reader - the next sublayer or the
model's last norm - folds it in, as ``NormedDelta`` does for a single stream.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import ops
from ..errors import ConfigError
from .base import CacheView, Param, Part, Piece
from .registry import register


@register("norm", "hyper_connection")
class HyperConnection(Part):
    """The three small tensors that tie one sublayer to the streams."""

    def __init__(self, streams: int):
        if not 1 <= streams <= 8:
            raise ConfigError(f"hyper_connection: {streams} streams are not built (1 to 8)")
        self.streams = streams
        self.in_weight = self.out_weight = self.mix_weight = None

    def params(self) -> List[Param]:
        S = self.streams
        return [Param("in_weight", (Piece("in", (S,)),), kind="vector", init="const:0.5"),
                Param("out_weight", (Piece("out", (S,)),), kind="vector", init="one_plus_normal"),
                Param("mix_weight", (Piece("mix", (S, S)),), kind="vector", init="identity")]


@dataclass
class HyperDelta:
    """A sublayer's output that is still to be written to the streams through ``connection``."""
    delta: torch.Tensor
    connection: HyperConnection


def streams_add_norm(norm, x: torch.Tensor, pending: Optional[HyperDelta], reader: Optional[HyperConnection],
                     rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Writes what is pending to the streams x [T, S, width] and returns norm(the reader's mixture of them) in the
    activation type; ``reader`` None mixes with ones (the sum of the streams).  With ``rows`` only those tokens are read and
    x is left as it is."""
    if not getattr(norm, "plain_rms", False):
        raise ConfigError("several residual streams are built with a plain RMS norm only")
    y = mix = out_w = None
    if pending is not None:
        if not isinstance(pending, HyperDelta):
            raise ConfigError("several residual streams: a sublayer's output must come with its connection")
        y, mix, out_w = pending.delta, pending.connection.mix_weight, pending.connection.out_weight
    return ops.hyper_step(x, y, mix, out_w, None if reader is None else reader.in_weight, norm.weight, norm.eps,
                          norm.act_dtype, rows)


class HyperBlock:
    """A pre-norm layer on several streams: mixer and (optional) feed-forward, each with a norm and a connection."""

    def __init__(self, norm1: Part, mixer: Part, hc1: HyperConnection, norm2: Optional[Part] = None,
                 feed_forward: Optional[Part] = None, hc2: Optional[HyperConnection] = None):
        self.norm1, self.mixer, self.hc1 = norm1, mixer, hc1
        self.norm2, self.feed_forward, self.hc2 = norm2, feed_forward, hc2

    def parts(self):
        p = {"norm1": self.norm1, "mixer": self.mixer, "hc1": self.hc1}
        if self.feed_forward is not None:
            p.update(norm2=self.norm2, feed_forward=self.feed_forward, hc2=self.hc2)
        return p

    def forward(self, x: torch.Tensor, pending, batch, cache):
        h = streams_add_norm(self.norm1, x, pending, self.hc1)
        pending = HyperDelta(self.mixer.forward(h, batch, cache), self.hc1)
        if self.feed_forward is None:
            return x, pending
        h = streams_add_norm(self.norm2, x, pending, self.hc2)
        return x, HyperDelta(self.feed_forward.forward(h, batch), self.hc2)
