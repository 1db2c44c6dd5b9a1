"""The Banazen design in the engine against the plain implementation of tests/plain_banazen.py: the new kernels against
torch arithmetic, each mixer and the feed-forward alone (one-layer models), whole models of several small shapes in every
cutting of requests into steps, batches against each request alone, keys just inside and just outside a window and far
back, a memory that must survive from step to step, long decoding through pages and slots that are used again, and greedy
generation through the entry points.

Routers: the float32 runs route by the data.  In bfloat16 the router's input differs from the float64 oracle's by the
rounding of the layers before it, enough to send some tokens to other experts than the oracle does; so the bfloat16 runs
of whole models choose all experts of a layer (the scores still differ from token to token), and data-dependent routing
in bfloat16 is covered by the router kernel's own test.
"""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fake_ops
import helpers
import plain_banazen as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = {"float32": 5e-5, "bfloat16": 6e-2}      # max |difference| / max |logit| over a step; float32 is the sharp test
STD = 0.12


def _lat(heads, dim, vdim, rank, scale, window=None, kv_from=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=rank, scale=scale)
    if window:
        m["mask"] = dict(size=window)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def _par(left, right):
    H, G, d, dv, scale, conv, rot = left
    l = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=scale, conv=conv)
    if rot:
        l["rot"] = dict(base=rot[0], dims=rot[1])
    r = dict(zip(("heads", "kv_heads", "dim", "vdim", "conv", "decay_rank", "gate_rank"), right))
    return dict(type="parallel", mixer=dict(left=l, right=r))


def _moe(ff, limit, experts, top, groups=(1, 1), scale=1.0, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff, limit=limit),
             router=dict(experts=experts, top=top, scale=scale, groups=dict(count=groups[0], keep=groups[1])))
    if shared:
        d["shared"] = dict(ff=shared[0], limit=shared[1])
    return d


def _dense(ff):
    return dict(kind="dense", ff=ff)


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def _model(vocab, width, layers, side=None, eps=1e-5, emb=1.0, logit_scale=1.0):
    d = dict(architecture="Banazen", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=emb),
             logit_scale=logit_scale, layers=layers)
    if side:
        d["token_side"] = dict(dim=side)
    return d


SHAPES = {
    # key and value sizes differ everywhere (the attention's heads are padded to 48 in the cache); a window of 24 positions,
    # no multiple of a page; a latent of 40 in a cache row of 48; a layer that reads another's latents through a window of
    # its own; 2 of 6 experts in 3 groups of which 2 stay; a dense layer; a layer without feed-forward; a rotation of half
    # of every head
    "a": _model(211, 96, [_layer(_par((4, 2, 32, 48, 0.2, 3, (100.0, 16)), (4, 2, 16, 24, 4, 6, 10)), _dense(64)),
                          _layer(_lat(3, 16, 24, 40, 0.3, window=24), _moe(24, 1.5, 6, 2, (3, 2), 1.7, (16, 0.8))),
                          _layer(_lat(5, 8, 8, 40, 0.5, window=9, kv_from=1), None),
                          _layer(_par((2, 2, 24, 16, 0.3, 1, None), (2, 1, 40, 20, 2, 3, 5)), _moe(40, 0.7, 4, 3))],
                side=10, emb=3.0, logit_scale=0.7),
    # nothing taken from the token, no scales; latent attention without a window first, then one with a window of one
    # page; full rotation; one query head per key/value head beside a delta rule with one key head for three
    "b": _model(300, 128, [_layer(_lat(2, 64, 64, 64, 0.125), _moe(64, 2.0, 8, 1, (4, 1), 2.5, (64, 1.0))),
                           _layer(_par((2, 2, 64, 64, 0.125, 4, (10000.0, 64)), (3, 1, 64, 32, 3, 8, 8)), None),
                           _layer(_lat(4, 32, 16, 128, 0.2, window=16), _dense(96)),
                           _layer(_lat(2, 16, 32, 128, 0.2, window=40, kv_from=2), _moe(32, 5.0, 6, 6, (2, 2), 0.8))], eps=1e-6),
    # awkward sizes: a width that is a multiple of 4 only, an odd vocabulary, heads of 20, 12, 24 and 40, a window of 7,
    # inner sizes that are no multiples of 8, a rotation of 6 dimensions, a token slice of 3
    "c": _model(203, 100, [_layer(_lat(5, 20, 12, 36, 0.4, window=7), _moe(28, 1.0, 9, 3, (3, 2), 1.2, (20, 2.5))),
                           _layer(_par((6, 2, 24, 40, 0.3, 2, (50.0, 6)), (4, 2, 20, 12, 4, 5, 7)), _moe(12, 3.0, 2, 2)),
                           _layer(_lat(2, 12, 20, 36, 0.3, kv_from=0), _dense(52))], side=3, eps=1e-4, emb=2.0, logit_scale=1.5),
}
SEEDS = {"a": 11, "b": 22, "c": 33}
LENGTHS = {"a": [1, 9, 33, 70, 150, 230], "b": [2, 17, 48, 97, 200], "c": [3, 40, 129, 75]}
# Requests are drawn from these seeds on.  (With 500, shape b's first request starts with a token whose delta-rule read-out
# at position 0, u (k . q), nearly cancels; the norm behind it blows the 16-bit rounding of q and k up to a third of the
# largest logit - in the torch doubles as in the kernels.  The float32 runs do not mind.)
REQUEST_SEEDS = {"a": 500, "b": 520, "c": 500}


def _raw(name, dtype):
    """The shape as tested in ``dtype``: in bfloat16 every routed layer chooses all of its experts."""
    raw = copy.deepcopy(SHAPES[name]) if isinstance(name, str) else copy.deepcopy(name)
    if dtype == "bfloat16":
        for layer in raw["layers"]:
            if layer["mlp"] and layer["mlp"]["kind"] == "moe":
                r = layer["mlp"]["router"]
                r["top"] = r["experts"]
                r["groups"]["keep"] = r["groups"]["count"]
    return raw


def _tensors(raw, seed, std=STD):
    from pico_vllm_b200.registry import config_from_dict
    from pico_vllm_b200.weights import random_tensors
    t = random_tensors(config_from_dict(raw), seed, std=std, dtype=torch.bfloat16)
    for n in t:         # norm weights around one, some well away from it; choice corrections large enough to change choices
        if (n.endswith(".norm") or n.endswith(".out") or n.endswith("norm1")) and t[n].dim() == 1:
            t[n] = (1.0 + 4.0 * (t[n].float() - 1.0)).to(torch.bfloat16)
        if n.endswith(".correction"):
            t[n] = (t[n].float() * 0.5).to(torch.bfloat16)
        if n.endswith(".A_log"):
            t[n] = (t[n].float() * 10.0 - 2.0).to(torch.bfloat16)      # decays from fast to slow
        if n.endswith(".conv"):
            t[n] = (t[n].float() * 1.5).to(torch.bfloat16)
        if ".mlp." in n and (n.endswith(".gate") or n.endswith(".up")):
            t[n] = (t[n].float() * 2.0).to(torch.bfloat16)             # so that the caps inside the experts cut
    return t


def _runner(raw, tensors, dtype, max_tokens, graph=False, page_size=16, max_num_seqs=4):
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache, model_from_tensors
    from pico_vllm_b200.registry import config_from_dict
    ecfg = EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=max_tokens, max_num_seqs=max_num_seqs,
                        use_cuda_graph=graph, device=DEV)
    model = model_from_tensors(config_from_dict(raw), tensors, ecfg)
    return ModelRunner(model, make_cache(model, ecfg, poison_freed=True), ecfg)


def _oracle(raw, tensors, reqs):
    return {rid: plain.forward(raw, tensors, ids) for rid, ids in reqs.items()}


def _compare(steps, reqs, got, logits, dtype, what):
    """float32, the sharp test: every step within REL of the plain implementation.  bfloat16: every wanted row's largest
    difference is measured against the largest logit of its step; all rows but a few (3% of the trace's, or one) stay within
    REL, and none is beyond five times that."""
    want = helpers.expected_logits(steps, reqs, logits)
    errs = []
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None), f"{what} step {i}"
        if w is None:
            continue
        assert g.shape == w.shape and torch.isfinite(g).all(), f"{what} step {i}: shape or a value that is not finite"
        if dtype == "float32":
            helpers.assert_close_logits(g, w.float(), REL[dtype], f"{what} step {i}")
        else:
            errs += [(float(e), i) for e in (g.double() - w.double()).abs().amax(1) / float(w.abs().max())]
    if errs:
        over = [(e, i) for e, i in errs if e > REL[dtype]]
        assert len(over) <= max(1, len(errs) * 3 // 100), f"{what}: {len(over)} of {len(errs)} rows over {REL[dtype]}: {over[:8]}"
        assert max(errs)[0] <= 5 * REL[dtype], f"{what}: a row is off by {max(errs)}"


def _shows(diff, scale, dtype):
    """Whether a difference between two oracles is large enough that the comparison in ``dtype`` would catch it."""
    return diff > max(20 * REL["float32"], 2 * REL[dtype]) * scale


def _status():
    from pico_vllm_b200 import ops
    ops.check_kernel_status()


# ------------------------------------------------------------------------------------------------ the kernels alone
def _segments(lens, pad_at=None):
    """cu_q, positions, tok_seg, seg_slots for segments of the given lengths (a segment ``pad_at`` is padding)."""
    cu, pos, seg = [0], [], []
    for s, n in enumerate(lens):
        cu.append(cu[-1] + n)
        pos += [-1] * n if s == pad_at else list(range(5 * s, 5 * s + n))
        seg += [s] * n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    return i32(cu), i32(pos), i32(seg), i32(list(range(len(lens) - 1, -1, -1)))


def _close(got, want, tol, what):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, what
    err = float((got - want).abs().max())
    assert err <= tol * max(1.0, float(want.abs().max())), f"{what}: off by {err}"


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 16, 24), (2, 2, 40, 8), (3, 1, 64, 64), (2, 1, 200, 130), (1, 1, 128, 16)])
@pytest.mark.parametrize("lens,pad_at", [([1, 70, 5, 2], 2), ([1, 1, 1], None), ([33], None)])
def test_delta_rule_kernels(H, G, d, dv, lens, pad_at):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(d + dv + len(lens))
    cu, pos, seg, slots = _segments(lens, pad_at)
    T, S = int(cu[-1]), len(lens)
    xc = torch.randn(T, 2 * G * d + H * dv + 3, generator=g)
    proj = torch.randn(T, H + 5, generator=g)
    dt = torch.randn(T, H * d, generator=g) * 2
    dt_bias, a_log = torch.randn(H * d, generator=g), torch.randn(H, generator=g) - 1.0
    for dtype in (torch.float32, torch.bfloat16):
        p, z = proj.to(dtype), dt.to(dtype)
        want = fake_ops.delta_prepare(xc, 2, 2 + G * d, p, 3, z, dt_bias, a_log, H, G, d)
        got = ops.delta_prepare(xc.to(DEV), 2, 2 + G * d, p.to(DEV), 3, z.to(DEV), dt_bias.to(DEV), a_log.to(DEV), H, G, d)
        _close(got, want, 2e-6, "delta_prepare")
    prep = want
    state = torch.randn(S + 1, H, dv, d, generator=g) * 0.3
    v = xc[:, 2 + 2 * G * d:]
    st_want = state.clone()
    o_want = fake_ops.gated_delta_rule(prep, v, st_want, slots, cu, pos, H, G, d, dv)
    st_got = state.to(DEV)
    o_got = ops.gated_delta_rule(prep.to(DEV), v.to(DEV), st_got, slots.to(DEV), cu.to(DEV), pos.to(DEV), H, G, d, dv)
    live = pos >= 0
    _close(o_got.cpu()[live], o_want[live], 2e-5, "delta rule outputs")
    _close(st_got, st_want, 2e-5, "delta rule states")
    _status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,rot,norm", [(4, 2, 32, 48, 16, True), (2, 2, 24, 16, 0, True), (6, 3, 64, 64, 64, False),
                                               (3, 1, 20, 12, 6, True)])
def test_pair_rope_norm_store(dtype, H, G, d, dv, rot, norm):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(d)
    T, ps, row = 11, 4, -(-max(d, dv) // 16) * 16
    x = torch.randn(T, (H + G) * d + G * dv + 1, generator=g)
    pos = torch.tensor([0, 1, 2, 300, 1117, -1, 7, 8, 9, 10, 11], dtype=torch.int32)
    slots = torch.tensor([0, 5, 6, 7, 9, -1, 13, -1, 20, 2, 31], dtype=torch.int32)
    inv = (37.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))).float() if rot else None
    qw, kw = (torch.rand(d, generator=g) + 0.5, None) if norm and d == 20 else (None, None)
    kp = torch.full((8, G, ps, row), float("nan")).to(dtype)
    vp = kp.clone()
    want = fake_ops.pair_rope_norm_store(x, 1, 1 + H * d, 1 + (H + G) * d, pos, inv, norm, qw, kw, 1e-5, slots, kp, vp, H, G, d, dv,
                                         row, ps, dtype)
    kg, vg = torch.full((8, G, ps, row), float("nan")).to(dtype).to(DEV), torch.full((8, G, ps, row), float("nan")).to(dtype).to(DEV)
    dev = lambda t: None if t is None else t.to(DEV)
    got = ops.pair_rope_norm_store(x.to(DEV), 1, 1 + H * d, 1 + (H + G) * d, pos.to(DEV), dev(inv), norm, dev(qw), dev(kw), 1e-5,
                                   slots.to(DEV), kg, vg, H, G, d, dv, row, ps, dtype)
    tol = 3e-4 if dtype == torch.float32 else 1e-2       # float32: the angle of position 1117 is rounded before sin and cos
    _close(got, want, tol, "queries")
    for a, b, what in ((kg, kp, "keys"), (vg, vp, "values")):
        assert torch.equal(torch.isnan(a.float().cpu()), torch.isnan(b.float()))      # nothing stored where nothing belongs
        _close(torch.nan_to_num(a.float()), torch.nan_to_num(b.float()), tol, what)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [96, 100, 2048, 4100])
def test_sum_add_norm(dtype, H):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(H)
    T = 9
    x = torch.randn(T, H, generator=g)
    ds = [torch.randn(T, H, generator=g).to(dtype) for _ in range(3)]
    ws = [torch.rand(H, generator=g) + 0.5 for _ in range(3)]
    cases = [[(ds[0], ws[0], 1, 1e-5, 0.5), (ds[1], ws[1], 1, 1e-4, 0.5), (ds[2], None, 0, 0.0, 1.0)],
             [(ds[0], None, 0, 0.0, 1.0), (ds[1], None, 0, 0.0, 1.0)], [(ds[2], None, 1, 1e-5, 2.0)], []]
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    for terms in cases:
        for kind, r in ((1, None), (3, None), (1, rows), (0, None)):
            if not terms and kind == 0:
                continue
            xw, xg = x.clone(), x.to(DEV)
            n = T if r is None else 3
            ow = torch.zeros(n, H).to(dtype) if kind else None
            og = torch.zeros(n, H).to(dtype).to(DEV) if kind else None
            fake_ops.sum_add_norm(xw, terms, ws[2], kind, 1e-5, ow, r)
            ops.sum_add_norm(xg, [(d.to(DEV), None if w is None else w.to(DEV), k, e, s) for d, w, k, e, s in terms], ws[2].to(DEV),
                             kind, 1e-5, og, None if r is None else r.to(DEV))
            _close(xg, xw, 1e-5, "stream")
            if kind:
                _close(og, ow, 1e-5 if dtype == torch.float32 else 1e-2, "handed on")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_gate_and_capped_activation(dtype):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(3)
    T, n, V = 13, 10, 17
    z = (torch.randn(T, n, generator=g) * 2).to(dtype)
    table = torch.randn(V, 4 * n + 3, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g).to(torch.int32)
    ids[4], ids[9] = -1, -2
    fb = torch.tensor([5, 11], dtype=torch.int32)
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    _close(ops.gelu_gate_rows(z.to(DEV), table.to(DEV), 2 * n + 1, ids.to(DEV), fb.to(DEV)),
           fake_ops.gelu_gate_rows(z, table, 2 * n + 1, ids, fb), tol, "token gate")
    for ff, limit, col in ((12, 0.7, None), (20, 2.0, 40), (7, 1.0, 15), (24, 1.3, 48), (64, 0.5, None)):
        gu = (torch.randn(T, 2 * ff + 8, generator=g) * 2).to(dtype)
        _close(ops.capped_glu(gu.to(DEV), ff, limit, col), fake_ops.capped_glu(gu, ff, limit, col), tol, "capped activation")


@pytest.mark.parametrize("E,top,groups,keep", [(6, 2, 3, 2), (16, 4, 4, 3), (8, 1, 4, 1), (9, 3, 3, 3), (12, 6, 1, 1), (40, 8, 8, 5)])
@pytest.mark.parametrize("T", [5, 700])
def test_router_with_groups_and_renormalised_weights(E, top, groups, keep, T):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(E + T)
    D = 72
    for dtype in (torch.float32, torch.bfloat16):
        h = torch.randn(T, D, generator=g).to(dtype)
        wr = torch.randn(E, D, generator=g) * 0.3
        corr = torch.randn(E, generator=g) * 0.3 - 0.2          # negative numbers among them: a group left out is not a zero
        wi, ww = fake_ops.moe_route(h, wr, None, top, 2, corr, 2.5, groups, keep, True)
        gi, gw = ops.moe_route(h.to(DEV), wr.to(DEV), None, top, ops.MOE_SCORE_SOFTMAX_ALL, corr.to(DEV), 2.5, groups, keep, True)
        same = (torch.sort(gi.cpu(), 1).values == torch.sort(wi, 1).values).all(1)
        assert float(same.float().mean()) > 0.99                # a near tie may fall the other way
        o1, o2 = torch.argsort(gi.cpu()[same], 1), torch.argsort(wi[same], 1)
        _close(torch.gather(gw.cpu()[same], 1, o1), torch.gather(ww[same], 1, o2), 1e-5, "weights")
        _close(gw.sum(1), torch.full((T,), 2.5), 1e-5, "the weights add up to the scale")


@pytest.mark.parametrize("dtype,T", [(torch.float32, 9), (torch.bfloat16, 9), (torch.bfloat16, 600)])
def test_capped_experts(dtype, T):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(T)
    D, ff, E, top = 64, 24, 5, 2
    h = torch.randn(T, D, generator=g).to(dtype)
    gu = (torch.randn(E, 2 * ff, D, generator=g) * 0.3).to(dtype)
    dn = (torch.randn(E, D, ff, generator=g) * 0.3).to(dtype)
    idx = torch.stack([torch.randperm(E - 1, generator=g)[:top] for _ in range(T)]).to(torch.int32)      # expert 4 gets nothing
    wgt = torch.rand(T, top, generator=g)
    base = torch.randn(T, D, generator=g).to(dtype)
    want = fake_ops.moe_experts(h, idx, wgt, gu, dn, True, 2, False, base, 0, 0.9)
    got = ops.moe_experts(h.to(DEV), idx.to(DEV), wgt.to(DEV), gu.to(DEV), dn.to(DEV), gated=True, act=ops.MOE_ACT_CAPPED,
                          base=base.to(DEV), limit=0.9)
    _close(got, want, 2e-5 if dtype == torch.float32 else 3e-2, "capped experts")


def test_convolution_without_activation_and_latent_store_without_query_part():
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(1)
    cu, pos, seg, slots = _segments([1, 9, 3, 2], 2)
    T, C, taps = int(cu[-1]), 40, 3
    proj = torch.randn(T, C + 4, generator=g)
    w = torch.randn(C, taps, generator=g)
    st = torch.randn(5, taps - 1, C, generator=g)
    for act in (False, True):
        sw, sg = st.clone(), st.to(DEV)
        want = fake_ops.causal_conv_silu(proj, 2, w, None, sw, seg, slots, cu, pos, act)
        got = ops.causal_conv_silu(proj.to(DEV), 2, w.to(DEV), None, sg, seg.to(DEV), slots.to(DEV), cu.to(DEV), pos.to(DEV), act=act)
        live = pos >= 0
        _close(got.cpu()[live], want[live], 2e-6, "convolution")
        _close(sg, sw, 1e-6, "its kept inputs")
    r, row = 20, 32
    p = torch.randn(T, r + 3, generator=g)
    kvw = torch.rand(r, generator=g) + 0.5
    rows = torch.tensor([3, 0, 9, -1, 7, 8, 1, 2, 30, 31, 12, 13, 14, 15, 16], dtype=torch.int32)
    cw, cg = torch.zeros(2, 1, 16, row), torch.zeros(2, 1, 16, row, device=DEV)
    fake_ops.latent_norm_store(p, 0, 0, None, 1, r, kvw, rows, cw, 0, 0, 1e-5)
    cq, gate = ops.latent_norm_store(p.to(DEV), 0, 0, None, 1, r, kvw.to(DEV), rows.to(DEV), cg, 0, 0, 1e-5)
    assert cq is None and gate is None
    _close(cg, cw, 2e-6, "latents")


# ------------------------------------------------------------------------------------------------ whole models
_CUTS = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decode(r, 32),
         "portions": helpers.trace_portions, "mixed": lambda r: helpers.trace_mixed(r, max_live=4, seed=3)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
@pytest.mark.parametrize("cut,graph", [("whole", False), ("tail", False), ("tail", True), ("portions", False),
                                       ("mixed", False), ("mixed", True)])
def test_every_cutting_matches_plain(dtype, name, cut, graph):
    raw = _raw(name, dtype)
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], REQUEST_SEEDS[name] + i) for i, n in enumerate(LENGTHS[name])}
    steps = _CUTS[cut](reqs)
    tensors = _tensors(raw, SEEDS[name])
    runner = _runner(raw, tensors, dtype, helpers.live_token_peak(steps), graph=graph)
    _compare(steps, reqs, helpers.replay(runner, steps), _oracle(raw, tensors, reqs), dtype, f"{name}/{cut}/{dtype}")
    if graph:
        assert runner.graph_replays > 0
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)      # every page came back
    _status()


def _random_shape(seed):
    """A model whose every size, count, constant and order of layers is drawn from ``seed``."""
    import random
    rnd = random.Random(seed)
    big = seed >= 8                           # from seed 8 on: heads of 128, latents of 256, more heads
    pick = lambda xs: rnd.choice(xs + xs[-1:] * 3) if big else rnd.choice(xs)
    width = pick([64, 72, 96, 160, 320])
    n = rnd.randint(3, 6)
    layers, makers = [], []                   # makers: layers that make their own latents (index, rank)
    for i in range(n):
        kind = pick(["parallel", "latent", "latent", "from"]) if makers else pick(["parallel", "latent"])
        if kind == "parallel":
            G = pick([1, 2, 3])
            H = G * pick([1, 2, 3])
            d, dv = pick([16, 32, 64, 24] + [128] * big), pick([16, 32, 64, 40] + [128] * big)
            rot = None if rnd.random() < 0.15 else (pick([100.0, 10000.0, 500000.0]), pick([d, d // 2, 8]))
            G2 = pick([1, 2, 4])
            right = (G2 * pick([1, 2]), G2, pick([16, 32, 64, 48] + [128] * big), pick([16, 32, 64, 24] + [128] * big), rnd.randint(1, 4),
                     rnd.randint(2, 12), rnd.randint(2, 12))
            mixer = _par((H, G, d, dv, pick([0.125, 0.2, d ** -0.5]), rnd.randint(1, 4), rot), right)
        else:
            window = pick([None, 5, 16, 33, 72, 100])
            H, d, dv = rnd.randint(1, 8) * (2 if big else 1), pick([16, 32, 64, 24] + [128] * big), pick([16, 32, 64, 8] + [128] * big)
            if kind == "from":
                src, rank = pick(makers)
                mixer = _lat(H, d, dv, rank, pick([0.125, 0.3]), window, kv_from=src)
            else:
                rank = pick([32, 64, 96, 128, 40] + [256] * big)
                makers.append((i, rank))
                mixer = _lat(H, d, dv, rank, pick([0.125, 0.3]), window)
        f = rnd.random()
        if f < 0.15:
            mlp = None
        elif f < 0.35:
            mlp = _dense(pick([48, 64, 100, 384]))
        else:
            count = pick([1, 2, 4])
            per = pick([1, 2, 4])
            keep = rnd.randint(1, count)
            top = rnd.randint(1, min(per * keep, 6))
            shared = None if rnd.random() < 0.3 else (pick([16, 40, 96]), pick([0.5, 1.0, 3.0]))
            mlp = _moe(pick([16, 24, 64]), pick([0.7, 2.0, 6.0]), count * per, top, (count, keep), pick([1.0, 2.5, 0.6]), shared)
        layers.append(_layer(mixer, mlp))
    return _model(pick([97, 211, 448, 1000]), width, layers, side=pick([None, 4, 24, 9]), eps=pick([1e-5, 1e-6, 1e-4]),
                  emb=pick([1.0, width ** 0.5, 0.3]), logit_scale=pick([1.0, 0.5, 2.0]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(12)))
def test_drawn_shapes_in_mixed_batches(dtype, seed):
    """Twelve models drawn at random - sizes, head counts, order of layers, windows, taps, groups, constants - each with four
    live requests, portions beside single tokens, pages and slots used again, against the plain implementation."""
    raw = _raw(_random_shape(seed), dtype)
    tensors = _tensors(raw, 100 + seed)
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 40 * seed + i) for i, n in enumerate([150, 3, 41, 77, 120, 18])}
    steps = helpers.trace_mixed(reqs, max_live=4, seed=seed)
    runner = _runner(raw, tensors, dtype, helpers.live_token_peak(steps), graph=seed % 2 == 0)
    _compare(steps, reqs, helpers.replay(runner, steps), _oracle(raw, tensors, reqs), dtype, f"drawn {seed}/{dtype}")
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)
    _status()


ALONE = {
    "latent": [_layer(_lat(3, 24, 40, 56, 0.3, window=20), None)],
    "many heads": [_layer(_lat(20, 16, 16, 32, 0.3, window=30), None), _layer(_lat(16, 24, 8, 32, 0.3, kv_from=0), None)],
    "shared latent": [_layer(_lat(2, 16, 16, 24, 0.3), None), _layer(_lat(4, 8, 24, 24, 0.4, window=11, kv_from=0), None)],
    "pair": [_layer(_par((4, 2, 32, 16, 0.4, 3, (1000.0, 20)), (3, 1, 24, 40, 4, 4, 6)), None)],
    "dense": [_layer(_lat(1, 8, 8, 16, 0.3), _dense(44))],
    "experts": [_layer(_lat(1, 8, 8, 16, 0.3), _moe(36, 0.6, 8, 3, (4, 2), 1.7, (52, 1.1)))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("side", [None, 6])
@pytest.mark.parametrize("what", sorted(ALONE))
def test_each_mechanism_alone(dtype, side, what):
    """A model of one layer (two for a layer that reads another's latents), with and without the part that reads the token:
    a whole prompt, then the same prompt token by token, then in portions down to two tokens."""
    raw = _raw(_model(157, 72, copy.deepcopy(ALONE[what]), side=side, emb=1.3), dtype)
    tensors = _tensors(raw, 5)
    reqs = {"p": helpers.random_ids(75, raw["vocab"], 21)}
    logits = _oracle(raw, tensors, reqs)
    for cut, steps in (("whole", helpers.trace_whole(reqs)), ("single", helpers.trace_tail_decode(reqs, 74)),
                       ("portions", helpers.trace_portions(reqs, sizes=(2, 5, 2, 21, 3)))):
        runner = _runner(raw, tensors, dtype, 128)
        _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"{what}/{cut}/{dtype}/{side}")
    _status()


def test_the_caps_and_the_groups_matter():
    """The oracle itself: without the caps inside the experts, without the groups, or with the correction in the weights the
    logits of the test shapes move by far more than the tolerance, so the whole-model tests would notice."""
    raw = _model(157, 72, copy.deepcopy(ALONE["experts"]), side=None)
    tensors = _tensors(raw, 5)
    ids = helpers.random_ids(40, raw["vocab"], 21)
    base = plain.forward(raw, tensors, ids)
    scale = float(base.abs().max())
    for change in ("limit", "shared limit", "groups"):
        other = copy.deepcopy(raw)
        f = other["layers"][0]["mlp"]
        if change == "limit":
            f["expert"]["limit"] = 50.0
        elif change == "shared limit":
            f["shared"]["limit"] = 50.0
        else:
            f["router"]["groups"] = dict(count=1, keep=1)
        assert _shows(float((plain.forward(other, tensors, ids) - base).abs().max()), scale, "float32"), change


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [4, 16, 64])
def test_other_page_sizes_and_batches_against_each_alone(dtype, page_size):
    """Unequal requests in one batch give what each gives alone (the same engine, one request per step), and both agree
    with the plain implementation."""
    raw = _raw("a", dtype)
    tensors = _tensors(raw, SEEDS["a"])
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 900 + i) for i, n in enumerate([6, 50, 17, 120])}
    together = [dict(entries=[dict(id=r, tokens=ids[:-4], want=list(range(len(ids) - 4))) for r, ids in reqs.items()], end=[])]
    for k in range(4, 0, -1):
        together.append(dict(entries=[dict(id=r, tokens=[ids[-k]], want=[0]) for r, ids in reqs.items()],
                             end=list(reqs) if k == 1 else []))
    alone = helpers.trace_tail_decode(reqs, 4)
    logits = _oracle(raw, tensors, reqs)
    outs = {}
    for what, steps in (("together", together), ("alone", alone)):
        runner = _runner(raw, tensors, dtype, helpers.live_token_peak(steps), page_size=page_size)
        got = helpers.replay(runner, steps)
        _compare(steps, reqs, got, logits, dtype, f"{what}/page {page_size}/{dtype}")
        at, rows = {r: 0 for r in reqs}, {}
        for st, g in zip(steps, got):
            i = 0
            for e in st["entries"]:
                for w in e["want"]:
                    rows[(e["id"], at[e["id"]] + w)] = g[i]
                    i += 1
                at[e["id"]] += len(e["tokens"])
        outs[what] = rows
    assert outs["together"].keys() == outs["alone"].keys()
    scale = max(float(v.abs().max()) for v in outs["alone"].values())
    worst = max(float((outs["together"][k] - outs["alone"][k]).abs().max()) for k in outs["alone"])
    assert worst <= (2e-5 if dtype == "float32" else 4e-2) * scale


def _sharp_latent(window):
    """One layer whose latent attention alone carries anything from token to token, with scores made sharp by a large
    factor on q.k."""
    return _model(97, 64, [_layer(_lat(4, 32, 32, 48, 6.0, window=window), None)])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [48, 50])
def test_keys_just_inside_and_just_outside_a_window(dtype, window):
    """A window of three pages and one that ends in the middle of a page.  The oracle with a window one longer or one shorter
    gives other logits by far more than the tolerance, so a window that is one token off shows; the engine must agree with
    the right one from a whole prompt, from single tokens and from portions cut at the window's length and at page borders."""
    raw = _sharp_latent(window)
    tensors = _tensors(raw, 91)
    ids = helpers.random_ids(4 * window + 9, raw["vocab"], 6)
    reqs = {"r": ids}
    logits = _oracle(raw, tensors, reqs)
    scale = float(logits["r"].abs().max())
    for other in (window - 1, window + 1):
        wrong = copy.deepcopy(raw)
        wrong["layers"][0]["mixer"]["mask"]["size"] = other
        diff = (plain.forward(wrong, tensors, ids) - logits["r"]).abs().amax(1)
        assert _shows(float(diff[window:].max()), scale, dtype)
    cuts = {"whole": helpers.trace_whole(reqs), "single": helpers.trace_tail_decode(reqs, 3 * window + 5),
            "edges": helpers.trace_portions(reqs, sizes=(window - 1, 2, window - 2, 3, window, window + 1, 2)),
            "pages": helpers.trace_portions(reqs, sizes=(16, 32, 15, 2, 48, 17))}
    for what, steps in cuts.items():
        runner = _runner(raw, tensors, dtype, 256)
        _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"{what}/{dtype}/window {window}")
    _status()


def _left_only(tensors):
    """The delta-rule side weighs nothing: the norm that follows it multiplies by zero."""
    for n in tensors:
        if n.endswith("right.out"):
            tensors[n] = torch.zeros_like(tensors[n])
    return tensors


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_and_the_first_tokens(dtype):
    """Causal attention behind the convolution over 420 equal tokens but one, at position 3.  The odd token is chosen so that
    the last queries prefer it; losing it (or the first inputs of the convolution) would show.  Read from a whole prompt,
    token by token, and in portions."""
    raw = _model(97, 64, [_layer(_par((2, 1, 32, 32, 8.0, 3, (10000.0, 8)), (1, 1, 8, 8, 2, 2, 2)), None)])
    tensors = _left_only(_tensors(raw, 17))
    base = [11] * 420
    plain_logits = plain.forward(raw, tensors, base)
    best, best_diff = None, 0.0
    for cand in range(20, 36):
        ids = list(base)
        ids[3] = cand
        d = float((plain.forward(raw, tensors, ids)[-1] - plain_logits[-1]).abs().max())
        if d > best_diff:
            best, best_diff = cand, d
    ids = list(base)
    ids[3] = best
    reqs = {"r": ids}
    logits = _oracle(raw, tensors, reqs)
    assert _shows(best_diff, float(logits["r"].abs().max()), dtype), best_diff
    cuts = {"whole": helpers.trace_whole(reqs), "single": helpers.trace_tail_decode(reqs, 200),
            "portions": helpers.trace_portions(reqs, sizes=(2, 2, 3, 64, 130, 2, 17))}
    for what, steps in cuts.items():
        runner = _runner(raw, tensors, dtype, 448)
        _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"{what}/{dtype}")
    _status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_memory_that_remembers_the_first_tokens(dtype):
    """The delta rule set to forget slowly, with keys of 64: the output at the end of 400 tokens still holds the first 200, so a
    memory that is lost, zeroed or handed to another request between steps shows.  Two requests take turns, in portions down to two tokens
    and single tokens, in slots that were used before; then whole prompts and long portions."""
    raw = _model(120, 64, [_layer(_par((4, 2, 32, 16, 0.4, 3, (1000.0, 20)), (3, 1, 64, 40, 4, 4, 6)), None)])
    tensors = _tensors(raw, 8)
    for n in tensors:
        if n.endswith(".A_log"):
            tensors[n] = torch.full_like(tensors[n], -9.0)
        if n.endswith("left.out"):
            tensors[n] = torch.zeros_like(tensors[n])                     # only the memory carries anything
    reqs = {"w": helpers.random_ids(40, raw["vocab"], 1), "x": helpers.random_ids(400, raw["vocab"], 2),
            "y": helpers.random_ids(300, raw["vocab"], 3)}
    logits = _oracle(raw, tensors, reqs)
    late = plain.forward(raw, tensors, [0] * 200 + reqs["x"][200:])     # other tokens in the first 200 places
    assert _shows(float((late[-1] - logits["x"][-1]).abs().max()), float(logits["x"].abs().max()), dtype)
    steps = helpers.trace_whole({"w": reqs["w"]})                         # uses a slot and gives it back
    steps += helpers.trace_mixed({"x": reqs["x"], "y": reqs["y"]}, max_live=2, seed=5, chunk_sizes=(2, 7, 64, 3, 2, 33))
    runner = _runner(raw, tensors, dtype, 1024, max_num_seqs=2)
    _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"memory/{dtype}")
    steps = helpers.trace_whole({"x": reqs["x"], "y": reqs["y"]}) + helpers.trace_portions({"x": reqs["x"]}, sizes=(300, 2, 98))
    _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"long portions/{dtype}")
    _status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_reused_slots(dtype):
    """300 single-token steps after a short prompt, twice, through a pool that holds one request."""
    raw = _raw("a", dtype)
    tensors = _tensors(raw, SEEDS["a"])
    reqs = {"x": helpers.random_ids(330, raw["vocab"], 41), "y": helpers.random_ids(330, raw["vocab"], 42)}
    steps = helpers.trace_tail_decode(reqs, 300)
    runner = _runner(raw, tensors, dtype, 384, graph=True, max_num_seqs=1)
    _compare(steps, reqs, helpers.replay(runner, steps), _oracle(raw, tensors, reqs), dtype, f"long decode/{dtype}")
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)
    _status()


# ------------------------------------------------------------------------------------------------ the entry points
def _greedy(raw, tensors, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(raw, tensors, ids)[-1].argmax()))
    return ids[len(prompt):]


def _write_model(raw, tensors, folder):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def test_greedy_generation_through_the_scheduler_and_the_command_line(tmp_path, capsys):
    """float32, so that the greedy choice is the oracle's: several requests of unequal length through ``LLM.generate`` (its
    scheduler cuts prompts into portions and batches them beside decoding requests), then one through the command line."""
    from pico_vllm_b200 import LLM, SamplingParams
    raw = SHAPES["c"]
    tensors = _tensors(raw, SEEDS["c"])
    folder = _write_model(raw, tensors, str(tmp_path / "model"))
    prompts = [helpers.random_ids(n, raw["vocab"], 70 + n) for n in (3, 41, 18, 77)]
    llm = LLM(folder, dtype="float32", page_size=16, max_cache_tokens=512, max_num_seqs=3, max_num_batched_tokens=32, device=DEV)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert list(o.token_ids) == _greedy(raw, tensors, p, 12)
    from pico_vllm_b200.cli import main
    capsys.readouterr()
    rc = main(["run", "--model", folder, "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompts[2])),
               "--prompt-ids", "9,9", "--max-new-tokens", "8", "--temperature", "0", "--num-gpu-blocks", "32", "--ignore-eos"])
    assert rc == 0
    lines = [l for l in capsys.readouterr().out.splitlines() if l.startswith("[")]
    printed = {int(l[1:l.index("]")]): [int(t) for t in l.split("] ")[1].split()] for l in lines}
    for rid, p in enumerate([prompts[2], [9, 9]]):       # prompt and generated tokens are printed together
        assert printed[rid] == p + _greedy(raw, tensors, p, 8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(tmp_path, dtype):
    """bin/trace_run on a model folder: four live requests, portions beside single tokens, pages and slots used again."""
    raw = _raw("a", dtype)
    tensors = _tensors(raw, SEEDS["a"])
    folder = _write_model(raw, tensors, str(tmp_path / "model"))
    reqs = {f"q{i}": helpers.random_ids(n, raw["vocab"], 300 + i) for i, n in enumerate([70, 5, 130, 33, 64, 90])}
    steps = helpers.trace_mixed(reqs, max_live=4, seed=9)
    out_dir = str(tmp_path / "out")
    lines = "".join(json.dumps(dict(step=i, **s)) + "\n" for i, s in enumerate(steps))
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
                          "--max-tokens", str(helpers.live_token_peak(steps))], input=lines, capture_output=True, text=True,
                         cwd=ROOT, timeout=1500)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [l for l in run.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    logits = _oracle(raw, tensors, reqs)
    got = [None if w is None else torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, raw["vocab"]))
           for i, w in enumerate(helpers.expected_logits(steps, reqs, logits))]
    _compare(steps, reqs, got, logits, dtype, f"trace_run/{dtype}")
