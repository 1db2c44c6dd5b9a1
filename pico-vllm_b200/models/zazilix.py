"""The Zazilix decoder put together from parts.

Embedding times a scale plus a learned vector per position; then layers on several residual streams (hyper-connections;
one plain pre-norm residual when the configuration has no ``streams``): RMS norm with a single learned number -> mixer ->
write to the streams, and the same with the feed-forward.  Mixers: the matrix memory with exponential gates, two mixers
side by side (chunked attention with a distance bias and a sink, and linear attention whose forget gate writes), or a
state-space layer.  Feed-forward: routed experts scored by a softmax over all router outputs, chosen with a correction,
some of them handing their input on, and a shared expert.  Last norm over the sum of the streams, an untied head.
Tensor names: ``embed``, ``pos``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.<in|out|mix>``, ``l<i>.mix.<...>`` (per mixer; the
two sides of a parallel mixer under ``left.`` and ``right.``), ``l<i>.mlp.<router|correction|e<k>.gate|e<k>.up|e<k>.down|
shared.gate|shared.up|shared.down>``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.zazilix import ZazilixConfig
from ..parts import (DistanceBiasAttention, ExpGatedMatrixMemory, ForgetWriteLinearAttention, HyperBlock, HyperConnection,
                     LearnedPositions, OutputHead, ParallelMixers, PreNormBlock, RoutedExperts, ScalarRMSNorm,
                     StateSpaceDuality, TokenEmbedding)
from .decoder import Binding, DecoderModel, LayerCall


def _w(prefix: str, *names: str):
    return {f"{n}.weight": prefix + n for n in names}


def _mixer(layer, D: int, eps: float, p: str):
    m = layer.mixer
    if layer.type == "mlstm":
        names = {**_w(p, "q", "k", "v", "g", "i", "f", "o"), "i.bias": p + "i.b", "f.bias": p + "f.b", "norm": p + "norm"}
        return ExpGatedMatrixMemory(D, m.heads, m.dim, m.vdim, m.gate_cap, eps), names
    if layer.type == "mamba2":
        names = {**_w(p, "in", "conv", "o"), "conv.bias": p + "conv.b", "dt_bias": p + "dt_bias", "A_log": p + "A_log",
                 "D": p + "D", "norm": p + "norm"}
        return StateSpaceDuality(D, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, eps), names
    l, r = m.left, m.right
    left = DistanceBiasAttention(D, l.heads, l.kv_heads, l.dim, l.vdim, eps, scale=l.scale, whole_qk_norm=True,
                                 value_norm=True, distance_bias=True, chunk=l.chunk, sink=0.0)
    right = ForgetWriteLinearAttention(D, r.heads, r.dim, r.vdim, eps)
    names = {f"left.{k}": v for k, v in {**_w(p + "left.", "q", "k", "v", "o"), "q.norm": p + "left.q.norm",
                                         "k.norm": p + "left.k.norm"}.items()}
    names.update({f"right.{k}": v for k, v in {**_w(p + "right.", "q", "f", "v", "o"), "f.bias": p + "right.f.b",
                                               "lower": p + "right.lower", "norm": p + "right.norm"}.items()})
    return ParallelMixers(left, right, m.left_scale, m.right_scale), names


def build_zazilix(cfg: ZazilixConfig) -> DecoderModel:
    D, eps, S = cfg.width, cfg.norm_eps, cfg.streams
    embed = TokenEmbedding(cfg.vocab, D)
    position = LearnedPositions(cfg.max_positions, D, input_scale=cfg.embedding_scale)
    bindings = [Binding(embed, {"weight": "embed"}), Binding(position, {"weight": "pos"})]
    blocks, order = [], []
    entries = 0
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mixer, names = _mixer(layer, D, eps, p + "mix.")
        norm1 = ScalarRMSNorm(D, eps)
        bindings += [Binding(norm1, {"weight": p + "norm1"}), Binding(mixer, names)]
        norm2 = ff = None
        if layer.mlp is not None:
            f = layer.mlp
            norm2 = ScalarRMSNorm(D, eps)
            ff = RoutedExperts(D, f.ff, f.experts, f.top, act="silu", router_bias=False, gated=True, scoring="softmax_all",
                               shared_inner=f.shared_ff, choice_bias=True, weight_scale=f.scale, identity=f.identity)
            ff_names = {"router.weight": p + "mlp.router", "correction": p + "mlp.correction"}
            for e in range(f.experts):
                ff_names.update({f"e{e}.{n}.weight": f"{p}mlp.e{e}.{n}" for n in ("gate", "up", "down")})
            if f.shared_ff:
                ff_names.update({f"shared.{n}.weight": f"{p}mlp.shared.{n}" for n in ("gate", "up", "down")})
            bindings += [Binding(norm2, {"weight": p + "norm2"}), Binding(ff, ff_names)]
        if S:
            hc1 = HyperConnection(S)
            bindings.append(Binding(hc1, {k: f"{p}hc1.{k}" for k in ("in", "out", "mix")}))
            hc2 = None
            if ff is not None:
                hc2 = HyperConnection(S)
                bindings.append(Binding(hc2, {k: f"{p}hc2.{k}" for k in ("in", "out", "mix")}))
            blocks.append(HyperBlock(norm1, mixer, hc1, norm2, ff, hc2))
        else:
            blocks.append(PreNormBlock(norm1, mixer, norm2, ff))
        spec = mixer.cache_spec()
        n = len(spec) if isinstance(spec, tuple) else 1
        ids = tuple(range(entries, entries + n))
        entries += n
        order.append(LayerCall(block=i, cache=ids if isinstance(spec, tuple) else ids[0]))
    final_norm = ScalarRMSNorm(D, eps)
    head = OutputHead(cfg.vocab, D)
    bindings += [Binding(final_norm, {"weight": "final.norm"}), Binding(head, {"weight": "head"})]
    return DecoderModel(cfg, embed, blocks, order, final_norm, head, bindings, embed_position=position, streams=S)
