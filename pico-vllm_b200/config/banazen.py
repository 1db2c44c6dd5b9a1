"""Configuration of the Banazen decoder, read from its config.json keys.

config.json names the model in ``architecture`` and describes the stack layer by layer: ``layers[i] = {"type": mixer kind,
"mixer": its sizes and constants, "mlp": its feed-forward or null}``.  Model-wide keys: ``vocab``, ``width``, ``norm.eps``,
``embedding.scale`` (on the token embedding; 1 when absent), ``logit_scale`` (1 when absent), ``token_side.dim`` (the
slice of a second embedding row that every layer reads; absent: layers take nothing from the token).  Mixer kinds:

* ``latent_attention`` - ``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``, ``mask.size`` (the window; absent: all keys),
  ``kv_from`` (an earlier layer whose cached latents this layer reads instead of making its own).
* ``parallel`` - ``left`` (attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``conv`` taps, ``rot.base`` and
  ``rot.dims``; no ``rot``: nothing is rotated) and ``right`` (delta rule: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv``;
  ``decay_rank`` and ``gate_rank``, the inner sizes of its two low-rank pairs, may be left out: the tensors have them).

Feed-forward: ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top",
"scale", "groups": {"count", "keep"}}, "shared": {"ff", "limit"} or absent}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..errors import ConfigError
from .base import KeyReader

ARCHITECTURE = "Banazen"
MIXER_KINDS = ("latent_attention", "parallel")


def _object(raw, at: str) -> KeyReader:
    if not isinstance(raw, dict):
        raise ConfigError(f"{at}: must be an object")
    return KeyReader(raw, at)


@dataclass(frozen=True)
class LatentSpec:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]
    kv_from: Optional[int]

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class ConvAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int
    rot_base: Optional[float]
    rot_dims: int

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "conv": self.conv}
        if self.rot_base is not None:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int] = None     # inner sizes of the two low-rank pairs: None = whatever the tensors have
    gate_rank: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.decay_rank is not None:
            d["decay_rank"] = self.decay_rank
        if self.gate_rank is not None:
            d["gate_rank"] = self.gate_rank
        return d


@dataclass(frozen=True)
class PairSpec:
    left: ConvAttentionSpec
    right: DeltaSpec

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                        # "dense" or "moe"
    ff: int
    limit: Optional[float] = None    # moe: the cap inside an expert
    experts: int = 0
    top: int = 0
    scale: float = 1.0
    groups: int = 1
    groups_keep: int = 1
    shared_ff: Optional[int] = None
    shared_limit: Optional[float] = None

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
             "router": {"experts": self.experts, "top": self.top, "scale": self.scale,
                        "groups": {"count": self.groups, "keep": self.groups_keep}}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: object
    mlp: Optional[FeedForwardSpec]

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class BanazenConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    side_dim: Optional[int]
    layers: Tuple[LayerSpec, ...]
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    max_position_embeddings: int = 1 << 20      # nothing in the design bounds a request's length

    architecture = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "BanazenConfig":
        r = KeyReader(raw, where)
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        eps = _object(r.any("norm"), f"{where}: norm").number("eps", positive=True)
        scale = 1.0 if r.any("embedding") is None else _object(r.any("embedding"), f"{where}: embedding").number("scale", default=1.0)
        side = None if r.any("token_side") is None else _object(r.any("token_side"), f"{where}: token_side").integer("dim", minimum=1)
        layers_raw = r.any("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        layers = []
        for i, item in enumerate(layers_raw):
            at = f"{where}: layers[{i}]"
            lr = _object(item, at)
            kind = lr.string("type")
            if kind == "latent_attention":
                mixer = _read_latent(lr.any("mixer"), f"{at}.mixer", i, layers)
            elif kind == "parallel":
                mixer = _read_pair(lr.any("mixer"), f"{at}.mixer")
            else:
                raise ConfigError(f"{at}: 'type' {kind!r} is not a mixer of {ARCHITECTURE} (have {list(MIXER_KINDS)})")
            layers.append(LayerSpec(kind, mixer, _read_ff(lr.any("mlp"), f"{at}.mlp")))
        dtype = r.string("torch_dtype", default=None) or r.string("dtype", default="bfloat16")
        return cls(vocab=vocab, width=width, norm_eps=eps, embedding_scale=scale,
                   logit_scale=r.number("logit_scale", default=1.0), side_dim=side, layers=tuple(layers), torch_dtype=dtype,
                   bos_token_id=r.integer("bos_token_id", default=None), eos_token_id=r.integer("eos_token_id", default=None))

    def to_dict(self) -> Dict[str, Any]:
        """config.json content that :meth:`from_dict` reads back to an equal object."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
             "layers": [l.to_dict() for l in self.layers]}
        if self.side_dim is not None:
            d["token_side"] = {"dim": self.side_dim}
        for k in ("bos_token_id", "eos_token_id"):
            if getattr(self, k) is not None:
                d[k] = getattr(self, k)
        return d


def _read_latent(raw, at: str, index: int, before) -> LatentSpec:
    m = _object(raw, at)
    window = None
    if m.any("mask") is not None:
        window = _object(m.any("mask"), f"{at}.mask").integer("size", minimum=1)
    spec = LatentSpec(m.integer("heads", minimum=1), m.integer("dim", minimum=1), m.integer("vdim", minimum=1),
                      m.integer("kv_rank", minimum=1), m.number("scale"), window, m.integer("kv_from", default=None, minimum=0))
    if spec.kv_from is not None:
        src = before[spec.kv_from] if spec.kv_from < index else None
        if src is None or src.type != "latent_attention" or src.mixer.kv_from is not None:
            raise ConfigError(f"{at}: 'kv_from' {spec.kv_from} must name an earlier latent_attention layer that makes its own latents")
        if src.mixer.kv_rank != spec.kv_rank:
            raise ConfigError(f"{at}: 'kv_rank' {spec.kv_rank} differs from the {src.mixer.kv_rank} of layer {spec.kv_from} whose latents it reads")
    return spec


def _read_pair(raw, at: str) -> PairSpec:
    m = _object(raw, at)
    l, r = _object(m.any("left"), f"{at}.left"), _object(m.any("right"), f"{at}.right")
    sides = []
    for s, where in ((l, f"{at}.left"), (r, f"{at}.right")):
        heads, kv_heads = s.integer("heads", minimum=1), s.integer("kv_heads", minimum=1)
        if heads % kv_heads:
            raise ConfigError(f"{where}: 'heads' {heads} must be a multiple of 'kv_heads' {kv_heads}")
        sides.append((heads, kv_heads, s.integer("dim", minimum=1), s.integer("vdim", minimum=1), s.integer("conv", default=1, minimum=1)))
    base, dims = None, 0
    if l.any("rot") is not None:
        rot = _object(l.any("rot"), f"{at}.left.rot")
        base, dims = rot.number("base", positive=True), rot.integer("dims", minimum=0)
        if dims % 2 or dims > sides[0][2]:
            raise ConfigError(f"{at}.left.rot: 'dims' {dims} must be even and at most 'dim' {sides[0][2]}")
    h, g, d, dv, conv = sides[0]
    left = ConvAttentionSpec(h, g, d, dv, l.number("scale"), conv, base, dims)
    return PairSpec(left, DeltaSpec(*sides[1], decay_rank=r.integer("decay_rank", default=None, minimum=1),
                                    gate_rank=r.integer("gate_rank", default=None, minimum=1)))


def _read_ff(raw, at: str) -> Optional[FeedForwardSpec]:
    if raw is None:
        return None
    f = _object(raw, at)
    kind = f.string("kind")
    if kind == "dense":
        return FeedForwardSpec("dense", f.integer("ff", minimum=1))
    if kind != "moe":
        raise ConfigError(f"{at}: 'kind' {kind!r} is not a feed-forward of {ARCHITECTURE} (have ['dense', 'moe'])")
    ex, rr = _object(f.any("expert"), f"{at}.expert"), _object(f.any("router"), f"{at}.router")
    experts, top = rr.integer("experts", minimum=1), rr.integer("top", minimum=1)
    count = keep = 1
    if rr.any("groups") is not None:
        g = _object(rr.any("groups"), f"{at}.router.groups")
        count = g.integer("count", minimum=1)
        keep = g.integer("keep", default=count, minimum=1)
    if experts % count or keep > count:
        raise ConfigError(f"{at}.router: {experts} experts do not form {count} equal groups of which {keep} are kept")
    if top > experts // count * keep:
        raise ConfigError(f"{at}.router: 'top' {top} exceeds the {experts // count * keep} experts of the kept groups")
    shared_ff = shared_limit = None
    if f.any("shared") is not None:
        sh = _object(f.any("shared"), f"{at}.shared")
        shared_ff, shared_limit = sh.integer("ff", minimum=1), sh.number("limit", positive=True)
    return FeedForwardSpec("moe", ex.integer("ff", minimum=1), ex.number("limit", positive=True), experts, top,
                           rr.number("scale", default=1.0), count, keep, shared_ff, shared_limit)
