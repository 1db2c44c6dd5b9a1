"""Configuration of the Zazilix decoder, read from its config.json keys.

config.json names the model in ``architecture`` and describes the stack layer by layer: ``layers[i] = {"type": mixer kind,
"mixer": its sizes and constants, "mlp": its feed-forward or null}``.  Model-wide keys: ``vocab``, ``width``, ``norm.eps``,
``embedding.scale`` (on the token embedding; 1 when absent), ``max_positions`` (rows of the learned position table),
``streams`` (residual streams per token; absent: one, the plain pre-norm residual).  Mixer kinds:

* ``mlstm`` - ``heads``, ``dim``, ``vdim``, ``gate_cap``.
* ``parallel`` - ``left`` (attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` the chunk of
  positions a query sees, absent: all before it), ``right`` (``heads``, ``dim``, ``vdim``), ``left_scale``, ``right_scale``.
* ``mamba2`` - ``heads``, ``vdim``, ``state``, ``groups``, ``conv`` (taps), ``norm_groups``.

Feed-forward: ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "identity"}, "shared": {"ff"} or
absent}``; ``identity`` router outputs after the experts' own hand their input on.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..errors import ConfigError
from .base import KeyReader

ARCHITECTURE = "Zazilix"
MIXER_KINDS = ("mlstm", "parallel", "mamba2")


def _object(raw, at: str) -> KeyReader:
    if not isinstance(raw, dict):
        raise ConfigError(f"{at}: must be an object")
    return KeyReader(raw, at)


@dataclass(frozen=True)
class MatrixMemorySpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class LeftSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        return d


@dataclass(frozen=True)
class RightSpec:
    heads: int
    dim: int
    vdim: int

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelSpec:
    left: LeftSpec
    right: RightSpec
    left_scale: float
    right_scale: float

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class StateSpaceSpec:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class ExpertsSpec:
    ff: int
    experts: int
    top: int
    scale: float
    identity: int
    shared_ff: Optional[int]

    def to_dict(self) -> Dict[str, Any]:
        d = {"kind": "moe", "expert": {"ff": self.ff},
             "router": {"experts": self.experts, "top": self.top, "scale": self.scale, "identity": self.identity}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: object
    mlp: Optional[ExpertsSpec]

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class ZazilixConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    max_positions: int
    streams: Optional[int]
    layers: Tuple[LayerSpec, ...]
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    architecture = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "ZazilixConfig":
        r = KeyReader(raw, where)
        vocab, width = r.integer("vocab", minimum=1), r.integer("width", minimum=1)
        eps = _object(r.any("norm"), f"{where}: norm").number("eps", positive=True)
        scale = 1.0 if r.any("embedding") is None else _object(r.any("embedding"), f"{where}: embedding").number("scale", default=1.0)
        streams = r.integer("streams", default=None, minimum=1)
        if streams is not None and streams > 8:
            raise ConfigError(f"{where}: 'streams' {streams} above 8 is not built")
        layers_raw = r.any("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        readers = {"mlstm": _read_memory, "parallel": _read_parallel, "mamba2": _read_state_space}
        layers = []
        for i, item in enumerate(layers_raw):
            at = f"{where}: layers[{i}]"
            lr = _object(item, at)
            kind = lr.string("type")
            if kind not in readers:
                raise ConfigError(f"{at}: 'type' {kind!r} is not a mixer of {ARCHITECTURE} (have {list(MIXER_KINDS)})")
            layers.append(LayerSpec(kind, readers[kind](lr.any("mixer"), f"{at}.mixer"), _read_ff(lr.any("mlp"), f"{at}.mlp")))
        dtype = r.string("torch_dtype", default=None) or r.string("dtype", default="bfloat16")
        return cls(vocab=vocab, width=width, norm_eps=eps, embedding_scale=scale,
                   max_positions=r.integer("max_positions", minimum=1), streams=streams, layers=tuple(layers),
                   torch_dtype=dtype, bos_token_id=r.integer("bos_token_id", default=None),
                   eos_token_id=r.integer("eos_token_id", default=None))

    def to_dict(self) -> Dict[str, Any]:
        """config.json content that :meth:`from_dict` reads back to an equal object."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "max_positions": self.max_positions,
             "layers": [l.to_dict() for l in self.layers]}
        if self.streams is not None:
            d["streams"] = self.streams
        for k in ("bos_token_id", "eos_token_id"):
            if getattr(self, k) is not None:
                d[k] = getattr(self, k)
        return d


def _read_memory(raw, at: str) -> MatrixMemorySpec:
    m = _object(raw, at)
    return MatrixMemorySpec(m.integer("heads", minimum=1), m.integer("dim", minimum=1), m.integer("vdim", minimum=1),
                            m.number("gate_cap", positive=True))


def _read_parallel(raw, at: str) -> ParallelSpec:
    m = _object(raw, at)
    l, r = _object(m.any("left"), f"{at}.left"), _object(m.any("right"), f"{at}.right")
    heads, kv_heads = l.integer("heads", minimum=1), l.integer("kv_heads", minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{at}.left: 'heads' {heads} must be a multiple of 'kv_heads' {kv_heads}")
    chunk = None
    if l.any("mask") is not None:
        chunk = _object(l.any("mask"), f"{at}.left.mask").integer("size", minimum=1)
    left = LeftSpec(heads, kv_heads, l.integer("dim", minimum=1), l.integer("vdim", minimum=1), l.number("scale"), chunk)
    right = RightSpec(r.integer("heads", minimum=1), r.integer("dim", minimum=1), r.integer("vdim", minimum=1))
    return ParallelSpec(left, right, m.number("left_scale", default=1.0), m.number("right_scale", default=1.0))


def _read_state_space(raw, at: str) -> StateSpaceSpec:
    m = _object(raw, at)
    s = StateSpaceSpec(m.integer("heads", minimum=1), m.integer("vdim", minimum=1), m.integer("state", minimum=1),
                       m.integer("groups", minimum=1), m.integer("conv", minimum=1), m.integer("norm_groups", default=1, minimum=1))
    if s.heads % s.groups:
        raise ConfigError(f"{at}: 'heads' {s.heads} must be a multiple of 'groups' {s.groups}")
    if (s.heads * s.vdim) % s.norm_groups:
        raise ConfigError(f"{at}: heads * vdim = {s.heads * s.vdim} must be a multiple of 'norm_groups' {s.norm_groups}")
    return s


def _read_ff(raw, at: str) -> Optional[ExpertsSpec]:
    if raw is None:
        return None
    f = _object(raw, at)
    kind = f.string("kind")
    if kind != "moe":
        raise ConfigError(f"{at}: 'kind' {kind!r} is not a feed-forward of {ARCHITECTURE} (have ['moe'])")
    rr = _object(f.any("router"), f"{at}.router")
    experts, top = rr.integer("experts", minimum=1), rr.integer("top", minimum=1)
    identity = rr.integer("identity", default=0, minimum=0)
    if top > experts + identity:
        raise ConfigError(f"{at}.router: 'top' {top} exceeds the {experts + identity} router outputs")
    shared = None
    if f.any("shared") is not None:
        shared = _object(f.any("shared"), f"{at}.shared").integer("ff", minimum=1)
    return ExpertsSpec(_object(f.any("expert"), f"{at}.expert").integer("ff", minimum=1), experts, top,
                       rr.number("scale", default=1.0), identity, shared)
