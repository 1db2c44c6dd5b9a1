"""The Banazen decoder put together from parts.

Embedding times a scale; then layers with ONE norm each: h = norm1(x); x += mixer(h) + feed_forward(h); and, when the model
has a second embedding table, x += norm(W_proj(gelu_tanh(W_gate x) * e)) with e the layer's slice of the token's row.
Mixers: latent attention over a window (queries projected directly, no gate; a layer with ``kv_from`` reads the latents an
earlier layer caches), or two mixers side by side - softmax attention behind a short convolution with rotated and normed
queries and keys, and the gated delta rule - each output RMS-normed, half their sum.  Feed-forward: dense, or routed experts
of the capped form (softmax scores, a correction for the choice, groups of experts, renormalised weights) with a gated shared
expert.  Last norm, an untied head, scaled logits.
Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1``, ``l<i>.mix.<q|dkv|dkv.norm|uk|uv|o>`` or ``l<i>.mix.left.<q|k|v|
q.conv|k.conv|v.conv|o|out>`` and ``l<i>.mix.right.<q|k|v|q.conv|k.conv|v.conv|b|a1|a2|dt_bias|A_log|g1|g2|norm|o|out>``,
``l<i>.mlp.<gate|up|down>`` or ``l<i>.mlp.<router|correction|e<k>.gate|e<k>.up|e<k>.down|shared.gate|shared.up|shared.down|
shared.sg>``, ``l<i>.side.<gate|proj|norm>``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.banazen import BanazenConfig
from ..parts import (ConvRopeAttention, GatedDeltaRule, GatedMLP, LatentAttention, OutputHead, ParallelBlock, ParallelMixers,
                     PassNorm, RMSNorm, RoutedExperts, TokenEmbedding, TokenSideInput, TokenSideTable)
from .decoder import Binding, DecoderModel, LayerCall


def _pair(m, D: int, eps: float, p: str):
    l, r = m.left, m.right
    left = ConvRopeAttention(D, l.heads, l.kv_heads, l.dim, l.vdim, eps, scale=l.scale, taps=l.conv, rot_base=l.rot_base,
                             rot_dim=l.rot_dims, qk_norm=True)
    right = GatedDeltaRule(D, r.heads, r.kv_heads, r.dim, r.vdim, r.conv, eps, r.decay_rank, r.gate_rank)
    names = {"left.out": p + "left.out", "right.out": p + "right.out"}
    for n in ("q", "k", "v", "o"):
        names[f"left.{n}.weight"] = f"{p}left.{n}"
    for n in ("q", "k", "v", "b", "a1", "a2", "g1", "g2", "o"):
        names[f"right.{n}.weight"] = f"{p}right.{n}"
    for side in ("left", "right"):
        for n in ("q", "k", "v"):
            names[f"{side}.{n}.conv"] = f"{p}{side}.{n}.conv"
    for n in ("dt_bias", "A_log", "norm"):
        names[f"right.{n}"] = f"{p}right.{n}"
    return ParallelMixers(left, right, 0.5, 0.5, left_norm=RMSNorm(D, eps), right_norm=RMSNorm(D, eps)), names


def _feed_forward(f, D: int, p: str):
    if f.kind == "dense":
        return GatedMLP(D, f.ff, "silu"), {f"{n}.weight": f"{p}{n}" for n in ("gate", "up", "down")}
    ff = RoutedExperts(D, f.ff, f.experts, f.top, act="capped", router_bias=False, gated=True, scoring="softmax_all",
                       shared_inner=f.shared_ff, choice_bias=True, weight_scale=f.scale, groups=f.groups,
                       groups_keep=f.groups_keep, renorm=True, limit=f.limit, shared_limit=f.shared_limit,
                       shared_gate=f.shared_ff is not None)
    names = {"router.weight": p + "router", "correction": p + "correction"}
    for e in range(f.experts):
        names.update({f"e{e}.{n}.weight": f"{p}e{e}.{n}" for n in ("gate", "up", "down")})
    if f.shared_ff:
        names.update({f"shared.{n}.weight": f"{p}shared.{n}" for n in ("gate", "up", "down", "sg")})
    return ff, names


def build_banazen(cfg: BanazenConfig) -> DecoderModel:
    D, eps = cfg.width, cfg.norm_eps
    embed = TokenEmbedding(cfg.vocab, D, scale=cfg.embedding_scale)
    bindings = [Binding(embed, {"weight": "embed"})]
    table = None
    if cfg.side_dim:
        table = TokenSideTable(cfg.vocab, len(cfg.layers), cfg.side_dim)
        bindings.append(Binding(table, {"weight": "side.embed"}))
    blocks, order = [], []
    entries = 0
    entry_of = {}                      # layer that keeps latents -> its cache entry
    keep = {}                          # ... -> how many latents its cache keeps: the longest window of its readers (None: all)
    for i, layer in enumerate(cfg.layers):
        if layer.type == "latent_attention":
            src = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            w = layer.mixer.window
            keep[src] = w if src not in keep else (None if w is None or keep[src] is None else max(w, keep[src]))
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "latent_attention":
            own = m.kv_from is None
            mixer = LatentAttention(D, m.heads, m.dim, m.vdim, None, m.kv_rank, m.scale, eps, own_latent=own, window=m.window,
                                    gate=False, cache_window=keep[i if own else m.kv_from])
            names = {"q.weight": p + "mix.q", "uk.weight": p + "mix.uk", "uv.weight": p + "mix.uv", "o.weight": p + "mix.o"}
            if own:
                names.update({"dkv.weight": p + "mix.dkv", "dkv.norm": p + "mix.dkv.norm"})
                entry_of[i] = entries
                entries += 1
            call = LayerCall(block=i, cache=entry_of[i if own else m.kv_from], store=own)
        else:
            mixer, names = _pair(m, D, eps, p + "mix.")
            n = len(mixer.cache_spec())
            call = LayerCall(block=i, cache=tuple(range(entries, entries + n)))
            entries += n
        norm1 = RMSNorm(D, eps)
        bindings += [Binding(norm1, {"weight": p + "norm1"}), Binding(mixer, names)]
        ff = None
        if layer.mlp is not None:
            ff, ff_names = _feed_forward(layer.mlp, D, p + "mlp.")
            bindings.append(Binding(ff, ff_names))
        side = None
        if table is not None:
            side_norm = RMSNorm(D, eps)
            side = TokenSideInput(D, cfg.side_dim, i, table, side_norm, PassNorm(D))
            bindings += [Binding(side, {"gate.weight": p + "side.gate", "proj.weight": p + "side.proj"}),
                         Binding(side_norm, {"weight": p + "side.norm"})]
        blocks.append(ParallelBlock(norm1, mixer, ff, side))
        order.append(call)
    final_norm = RMSNorm(D, eps)
    head = OutputHead(cfg.vocab, D, logit_scale=cfg.logit_scale)
    bindings += [Binding(final_norm, {"weight": "final.norm"}), Binding(head, {"weight": "head"})]
    return DecoderModel(cfg, embed, blocks, order, final_norm, head, bindings)
