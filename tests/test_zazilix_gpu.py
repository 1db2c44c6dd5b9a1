"""The Zazilix design in the engine against the plain implementation of tests/plain_zazilix.py: each mixer and the
feed-forward alone (one-layer models, with one residual stream and with several), whole models of several small shapes in
every cutting of requests into steps, batches against each request alone, keys just inside and just outside a chunk and
far back, states that must survive from step to step, long decoding through pages and slots that are used again, the new
kernels against torch arithmetic, and greedy generation through the entry points.

Routers: the float32 runs route by the data.  In bfloat16 the router's input differs from the float64 oracle's by the
rounding of the layers before it, enough to send some tokens to other experts than the oracle does; so the bfloat16 runs
of whole models choose all router outputs of a layer (the scores still differ from token to token), and data-dependent
routing in bfloat16 is covered by the router kernel's own test.
"""
import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_zazilix as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = {"float32": 5e-5, "bfloat16": 6e-2}      # max |difference| / max |logit| over a step; float32 is the sharp test
STD = 0.12


def _mem(heads, dim, vdim, cap=8.0):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap))


def _par(left, right, ls=0.7, rs=0.4):
    H, G, d, dv, scale, chunk = left
    l = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=scale)
    if chunk:
        l["mask"] = dict(size=chunk)
    return dict(type="parallel", mixer=dict(left=l, right=dict(zip(("heads", "dim", "vdim"), right)), left_scale=ls, right_scale=rs))


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return dict(type="mamba2", mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups))


def _moe(ff, experts, top, identity=0, scale=1.0, shared=None):
    d = dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale, identity=identity))
    if shared:
        d["shared"] = dict(ff=shared)
    return d


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def _model(vocab, width, layers, streams=None, eps=1e-5, emb=1.0, positions=1024):
    d = dict(architecture="Zazilix", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=emb),
             max_positions=positions, layers=layers)
    if streams:
        d["streams"] = streams
    return d


SHAPES = {
    # three streams; key and value sizes differ everywhere (the attention's heads are padded to 48 in the cache); a chunk of
    # 24 positions, no multiple of a page; 2 of 5 + 1 router outputs with a shared expert; a layer without feed-forward;
    # all 3 of 3 experts, none that hands its input on, no shared one
    "a": _model(211, 96, [_layer(_par((4, 2, 32, 48, 0.2, 24), (3, 16, 24)), _moe(40, 5, 2, identity=1, scale=1.5, shared=24)),
                          _layer(_mem(3, 16, 24), None),
                          _layer(_ssm(4, 16, 16, 2, 3, 2), _moe(24, 3, 3))], streams=3, emb=0.7),
    # one residual stream (the plain pre-norm layer); starts with the state-space layer: one group, one norm part, keys of
    # 64; a memory with heads of 64; attention without a chunk, one query head per key/value head, beside one wide head
    "b": _model(300, 128, [_layer(_ssm(2, 64, 64, 1, 4, 1), _moe(64, 4, 1, identity=2, scale=2.5, shared=64)),
                           _layer(_mem(2, 64, 64, cap=15.0), _moe(32, 6, 3, scale=0.8)),
                           _layer(_par((2, 2, 64, 64, 0.125, None), (1, 128, 32), ls=1.0, rs=1.0), None)], eps=1e-6),
    # awkward sizes: a width that is a multiple of 4 only, an odd vocabulary, heads of 20, 12, 24 and 40, a chunk of 7, a
    # convolution of 2 taps, 3 groups and 3 norm parts, inner sizes that are no multiples of 8, eight streams
    "c": _model(203, 100, [_layer(_mem(5, 20, 12, cap=5.0), _moe(28, 7, 3, identity=2, scale=1.2, shared=20)),
                           _layer(_par((6, 2, 24, 40, 0.3, 7), (2, 40, 20), ls=0.5, rs=1.5), _moe(12, 2, 2, identity=1)),
                           _layer(_ssm(3, 20, 24, 3, 2, 3), None)], streams=8, eps=1e-4, emb=2.0),
    # sizes that are multiples of 2 at most, two streams, a convolution of one tap (no inputs kept), a chunk of one page
    "d": _model(101, 90, [_layer(_ssm(2, 6, 10, 2, 1, 1), _moe(10, 2, 1, shared=6)),
                          _layer(_par((3, 1, 16, 16, 0.5, 16), (2, 8, 4)), _moe(14, 3, 2, identity=1, scale=3.0)),
                          _layer(_mem(2, 8, 4), None)], streams=2),
}
SEEDS = {"a": 11, "b": 22, "c": 33, "d": 44}
LENGTHS = {"a": [1, 9, 33, 70, 150, 230], "b": [2, 17, 48, 97, 200], "c": [3, 40, 129, 75], "d": [5, 60, 300]}


def _raw(name, dtype):
    """The shape as tested in ``dtype``: in bfloat16 every routed layer chooses all of its router outputs."""
    raw = copy.deepcopy(SHAPES[name])
    if dtype == "bfloat16":
        for layer in raw["layers"]:
            if layer["mlp"]:
                r = layer["mlp"]["router"]
                r["top"] = r["experts"] + r["identity"]
    return raw


def _tensors(raw, seed, std=STD):
    from pico_vllm_b200.registry import config_from_dict
    from pico_vllm_b200.weights import random_tensors
    t = random_tensors(config_from_dict(raw), seed, std=std, dtype=torch.bfloat16)
    for n in t:         # norm weights around one, some well away from it; choice corrections large enough to change choices
        if n.endswith(".norm") and t[n].dim() == 1:
            t[n] = (1.0 + 4.0 * (t[n].float() - 1.0)).to(torch.bfloat16)
        if n.endswith(".correction"):
            t[n] = (t[n].float() * 0.5).to(torch.bfloat16)
        if n.endswith(".A_log"):
            t[n] = (t[n].float() * 10.0 - 1.5).to(torch.bfloat16)      # decays from fast to slow
        if n.endswith("mix.f.b"):
            t[n] = (t[n].float() * 10.0 + 2.0).to(torch.bfloat16)      # forget gates of the memory that keep most
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


def _greedy(raw, tensors, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(raw, tensors, ids)[-1].argmax()))
    return ids[len(prompt):]


def _compare(steps, reqs, got, logits, dtype, what):
    """float32, the sharp test: every step within REL of the plain implementation.  bfloat16: every wanted row's largest
    difference is measured against the largest logit of its step; all rows but a few (3% of the trace's, or one) stay within
    REL, and none is beyond five times that.  The few: a head whose output nearly cancels is blown up to unit size by the
    norm that follows it, and with it the rounding of its 16-bit inputs; the float64 oracle has no such token."""
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


_CUTS = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decode(r, 32),
         "portions": helpers.trace_portions, "mixed": lambda r: helpers.trace_mixed(r, max_live=4, seed=3)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
@pytest.mark.parametrize("cut,graph", [("whole", False), ("tail", False), ("tail", True), ("portions", False),
                                       ("mixed", False), ("mixed", True)])
def test_every_cutting_matches_plain(dtype, name, cut, graph):
    raw = _raw(name, dtype)
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 500 + i) for i, n in enumerate(LENGTHS[name])}
    steps = _CUTS[cut](reqs)
    tensors = _tensors(raw, SEEDS[name])
    runner = _runner(raw, tensors, dtype, helpers.live_token_peak(steps), graph=graph)
    _compare(steps, reqs, helpers.replay(runner, steps), _oracle(raw, tensors, reqs), dtype, f"{name}/{cut}/{dtype}")
    if graph:
        assert runner.graph_replays > 0
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)      # every page came back
    _status()


ALONE = {
    "memory": [_layer(_mem(3, 24, 40, cap=6.0), None)],
    "attention": [_layer(_par((4, 2, 32, 16, 0.4, 20), (1, 8, 8), ls=1.0, rs=0.0), None)],
    "forget-write": [_layer(_par((1, 1, 16, 16, 0.1, 4), (3, 24, 40), ls=0.0, rs=1.0), None)],
    "state space": [_layer(_ssm(6, 24, 40, 3, 5, 2), None)],
    "experts": [_layer(_mem(1, 8, 8), _moe(36, 6, 3, identity=2, scale=1.7, shared=52))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("streams", [None, 4])
@pytest.mark.parametrize("what", sorted(ALONE))
def test_each_mechanism_alone(dtype, streams, what):
    """A model of one layer with one kind of mixer (the other side of a parallel mixer weighs nothing), on one residual
    stream and on four: a whole prompt, then the same prompt token by token, then in portions down to two tokens."""
    raw = _model(157, 72, copy.deepcopy(ALONE[what]), streams=streams, emb=1.3)
    if dtype == "bfloat16" and what == "experts":
        raw["layers"][0]["mlp"]["router"]["top"] = 8
    tensors = _tensors(raw, 5)
    reqs = {"p": helpers.random_ids(75, raw["vocab"], 21)}
    logits = _oracle(raw, tensors, reqs)
    for cut, steps in (("whole", helpers.trace_whole(reqs)), ("single", helpers.trace_tail_decode(reqs, 74)),
                       ("portions", helpers.trace_portions(reqs, sizes=(2, 5, 2, 21, 3)))):
        runner = _runner(raw, tensors, dtype, 128)
        _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"{what}/{cut}/{dtype}/{streams}")
    _status()


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


def _sharp_attention(chunk, heads=4, kv_heads=2):
    """One layer whose attention alone carries anything from token to token (the linear side weighs nothing, there is no
    feed-forward), with scores made sharp by a large factor on q.k."""
    return _model(97, 64, [_layer(_par((heads, kv_heads, 32, 32, 1.2, chunk), (1, 8, 8), ls=1.0, rs=0.0), None)], streams=2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [48, 50])
def test_keys_just_inside_and_just_outside_a_chunk(dtype, chunk):
    """A chunk of three pages and one that ends in the middle of a page.  The oracle with a chunk one longer or one shorter
    gives other logits at the chunks' edges by far more than the tolerance, so a window that is one token off shows; the
    engine must agree with the right one from a whole prompt, from single tokens and from portions cut at the edges."""
    raw = _sharp_attention(chunk)
    tensors = _tensors(raw, 91)
    ids = helpers.random_ids(4 * chunk + 9, raw["vocab"], 6)
    reqs = {"r": ids}
    logits = _oracle(raw, tensors, reqs)
    scale = float(logits["r"].abs().max())
    for other in (chunk - 1, chunk + 1):
        wrong = copy.deepcopy(raw)
        wrong["layers"][0]["mixer"]["left"]["mask"]["size"] = other
        diff = (plain.forward(wrong, tensors, ids) - logits["r"]).abs().amax(1)
        edges = [k * chunk + e for k in range(1, 4) for e in (-1, 0)]
        assert _shows(float(diff[edges].max()), scale, dtype)
    cuts = {"whole": helpers.trace_whole(reqs), "single": helpers.trace_tail_decode(reqs, 3 * chunk + 5),
            "edges": helpers.trace_portions(reqs, sizes=(chunk - 1, 2, chunk - 2, 3, chunk, chunk + 1, 2)),
            "pages": helpers.trace_portions(reqs, sizes=(16, 32, 15, 2, 48, 17))}
    for what, steps in cuts.items():
        runner = _runner(raw, tensors, dtype, 256)
        _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"{what}/{dtype}/chunk {chunk}")
    _status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_and_the_first_tokens(dtype):
    """Attention without a chunk over 420 equal tokens but one, at position 3, with no learned positions: the keys differ in
    that one place only.  The odd token is chosen so that the last queries prefer it; losing it, or the distance bias, or
    the sink would show.  Read from a whole prompt, token by token, and in portions."""
    raw = _sharp_attention(None, heads=2, kv_heads=1)
    tensors = _tensors(raw, 17)
    tensors["pos"] = torch.zeros_like(tensors["pos"])
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
    # the first tokens: with a sink of score 0 the first position's weight is well below one
    cuts = {"whole": helpers.trace_whole(reqs), "single": helpers.trace_tail_decode(reqs, 200),
            "portions": helpers.trace_portions(reqs, sizes=(2, 2, 3, 64, 130, 2, 17))}
    for what, steps in cuts.items():
        runner = _runner(raw, tensors, dtype, 448)
        _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"{what}/{dtype}")
    _status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["memory", "forget-write", "state space"])
def test_a_state_that_remembers_the_first_tokens(dtype, kind):
    """One recurrent layer set to forget slowly: the output at the end of 500 tokens still holds the first 150, so a state
    that is lost, zeroed or handed to another request between steps shows.  Two requests take turns, in portions down to two
    tokens and single tokens, in slots that were used before; then whole prompts (the chunks of a long portion run side by
    side with a scan between them) and long portions."""
    raw = _model(120, 64, copy.deepcopy(ALONE[kind]), streams=2)
    if kind == "memory":
        raw["layers"][0]["mixer"]["gate_cap"] = 20.0                        # a cap that lets the forget gate come close to one
    tensors = _tensors(raw, 8)
    for n in tensors:
        if n.endswith("mix.f.b"):
            tensors[n] = torch.full_like(tensors[n], 6.0)               # the memory forgets about 1/400 a token
        if n.endswith("right.lower"):
            tensors[n] = torch.full_like(tensors[n], 0.996)
        if n.endswith(".A_log"):
            tensors[n] = torch.full_like(tensors[n], -5.5)
    reqs = {"w": helpers.random_ids(40, raw["vocab"], 1), "x": helpers.random_ids(500, raw["vocab"], 2),
            "y": helpers.random_ids(300, raw["vocab"], 3)}
    logits = _oracle(raw, tensors, reqs)
    late = plain.forward(raw, tensors, [0] * 150 + reqs["x"][150:])     # other tokens in the first 150 places
    assert _shows(float((late[-1] - logits["x"][-1]).abs().max()), float(logits["x"].abs().max()), dtype)
    steps = helpers.trace_whole({"w": reqs["w"]})                         # uses a slot and gives it back
    steps += helpers.trace_mixed({"x": reqs["x"], "y": reqs["y"]}, max_live=2, seed=5, chunk_sizes=(2, 7, 64, 3, 2, 33))
    runner = _runner(raw, tensors, dtype, 1024, max_num_seqs=2)
    _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"state/{kind}/{dtype}")
    steps = helpers.trace_whole({"x": reqs["x"], "y": reqs["y"]}) + helpers.trace_portions({"x": reqs["x"]}, sizes=(300, 2, 198))
    _compare(steps, reqs, helpers.replay(runner, steps), logits, dtype, f"long portions/{kind}/{dtype}")
    _status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_reused_slots(dtype):
    """300 single-token steps after a short prompt, twice, through a pool that holds one request."""
    raw = _raw("a", dtype)
    tensors = _tensors(raw, SEEDS["a"])
    reqs = {"x": helpers.random_ids(330, raw["vocab"], 41), "y": helpers.random_ids(330, raw["vocab"], 42)}
    steps = helpers.trace_tail_decode(reqs, 300)
    runner = _runner(raw, tensors, dtype, 384, graph=True, max_num_seqs=1)
    _compare(steps, reqs, helpers.replay(runner, steps), _oracle(raw, tensors, reqs), dtype, f"long/{dtype}")
    assert runner.graph_replays > 500
    _status()


# ------------------------------------------------------------------ the kernels alone, against torch arithmetic
def _close(got, want, dtype, what):
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    err = float((got.double().cpu() - want.double().cpu()).abs().max())
    assert err <= tol * max(1.0, float(want.abs().max())), f"{what}: {err}"


@pytest.mark.parametrize("H,rep,d,dv", [(3, 1, 16, 24), (4, 2, 64, 16), (1, 1, 20, 13), (6, 3, 40, 70), (2, 1, 200, 33), (2, 1, 24, 65),
                                        (3, 1, 128, 129)])
@pytest.mark.parametrize("per_row", [False, True])
@pytest.mark.parametrize("chunk", [0, 16, 3])
def test_gated_recurrence_kernel(H, rep, d, dv, per_row, chunk):
    """Segments of 1, 70, 2, 9 and 8 tokens and a padding segment, from states that are not zero, into slots in any order;
    walked token by token (chunk 0) or as chunks side by side with a scan between them; q, k, v and the gates are column
    slices of wider rows."""
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(d * 7 + dv + H)
    lens = [1, 70, 2, 9, 8, 1]
    T = sum(lens)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    pos = torch.arange(T, dtype=torch.int32)
    pos[cu[5]:] = -1
    seg_slots = torch.tensor([4, 0, 6, 2, 5, 0], dtype=torch.int32)
    G = H // rep
    wide = torch.randn(T, 2 * G * d + H * dv + 5, generator=g) * 0.7
    q, k, v = wide[:, :G * d], wide[:, G * d:2 * G * d], wide[:, 2 * G * d:2 * G * d + H * dv]
    gate = torch.rand(T, (H * d if per_row else H) + 3, generator=g)[:, 3:] * 0.6 + 0.4
    state = torch.randn(7, H, dv, d, generator=g) * 0.3
    want_state = state.clone().double()
    want = torch.zeros(T, H * dv, dtype=torch.float64)
    for s in range(5):
        for h in range(H):
            S = want_state[seg_slots[s], h].T.clone()                     # [d, dv]
            for t in range(int(cu[s]), int(cu[s + 1])):
                a = gate[t, h * d:(h + 1) * d].double()[:, None] if per_row else float(gate[t, h])
                kk, qq = k[t, (h // rep) * d:(h // rep + 1) * d].double(), q[t, (h // rep) * d:(h // rep + 1) * d].double()
                S = a * S + torch.outer(kk, v[t, h * dv:(h + 1) * dv].double())
                want[t, h * dv:(h + 1) * dv] = S.T @ qq
            want_state[seg_slots[s], h] = S.T
    dev = lambda t: t.to(DEV)
    wd, gd, st = dev(wide), dev(torch.cat([torch.zeros(T, 3), gate], 1)), dev(state)
    out = ops.gated_linear_attention(wd[:, :G * d], wd[:, G * d:2 * G * d], wd[:, 2 * G * d:2 * G * d + H * dv], gd[:, 3:], per_row,
                                     st, dev(seg_slots), dev(cu), dev(pos), H, rep, d, dv, max_q_len=70, chunk=chunk)
    live = pos >= 0
    _close(out[live.to(DEV)], want[live], torch.float32, "outputs")
    _close(st, want_state, torch.float32, "states")
    _status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,D", [(1, 64), (4, 100), (8, 2048), (3, 6)])
def test_streams_kernels(dtype, S, D):
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(S * 10 + D)
    T = 19
    x = torch.randn(T, S, D, generator=g)
    y = torch.randn(T, D, generator=g).to(dtype)
    mix, ow, iw = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    nw = torch.rand(D, generator=g) + 0.5
    new = torch.einsum("sr,tsd->trd", mix.double(), x.double()) + ow.double()[None, :, None] * y.double()[:, None, :]
    u = torch.einsum("s,tsd->td", iw.double(), new)
    want = u / torch.sqrt((u * u).mean(-1, keepdim=True) + 1e-5) * nw.double()
    xd = x.to(DEV)
    h = ops.hyper_step(xd, y.to(DEV), mix.to(DEV), ow.to(DEV), iw.to(DEV), nw.to(DEV), 1e-5, dtype)
    _close(h, want, dtype, "read after write")
    _close(xd, new, torch.float32, "streams")
    rows = torch.tensor([3, 0, 18], dtype=torch.int32)
    x2 = x.to(DEV)
    h = ops.hyper_step(x2, y.to(DEV), mix.to(DEV), ow.to(DEV), None, nw.to(DEV), 1e-5, dtype, rows=rows.to(DEV))
    s = new.sum(1)[rows.long()]
    _close(h, s / torch.sqrt((s * s).mean(-1, keepdim=True) + 1e-5) * nw.double(), dtype, "sum of some rows")
    assert torch.equal(x2.cpu(), x)                                       # rows given: nothing is written
    h = ops.hyper_step(x2, None, None, None, iw.to(DEV), nw.to(DEV), 1e-5, dtype)
    u = torch.einsum("s,tsd->td", iw.double(), x.double())
    _close(h, u / torch.sqrt((u * u).mean(-1, keepdim=True) + 1e-5) * nw.double(), dtype, "read alone")
    e = torch.randn(T, D, generator=g)
    assert torch.equal(ops.hyper_expand(e.to(DEV), S).cpu(), e[:, None, :].expand(T, S, D))
    table = torch.randn(50, D, generator=g).to(dtype)
    p = torch.randint(0, 50, (T,), generator=g).to(torch.int32)
    p[4] = -1
    want = e.double() * 0.3 + torch.where((p >= 0)[:, None], table.double()[p.clamp(min=0).long()], torch.zeros(1, dtype=torch.float64))
    _close(ops.scale_add_rows(e.to(DEV), 0.3, table.to(DEV), p.to(DEV)), want, torch.float32, "scale and positions")
    a, b = torch.randn(T, D, generator=g).to(dtype), torch.randn(T, D, generator=g).to(dtype)
    _close(ops.scaled_sum(a.to(DEV), 0.6, b.to(DEV), -1.5), 0.6 * a.double() - 1.5 * b.double(), dtype, "scaled sum")
    _status()


@pytest.mark.parametrize("E,ident,top", [(5, 1, 2), (16, 0, 4), (3, 2, 5), (40, 3, 6)])
def test_router_over_all_outputs_with_a_choice_correction(E, ident, top):
    """The scores are the softmax over all outputs; the choice adds the correction, the weights do not; and the sum of the
    experts' outputs passes the input on for the outputs beyond the real experts."""
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(E + top)
    T, D, ff = 33, 48, 24
    for dtype in (torch.float32, torch.bfloat16):
        h = torch.randn(T, D, generator=g).to(dtype)
        wr = torch.randn(E + ident, D, generator=g) * 0.5
        corr = torch.randn(E + ident, generator=g) * 0.2
        s = torch.softmax(h.double() @ wr.double().T, -1)
        chosen = torch.topk(s + corr.double(), top, dim=-1).indices
        idx, wgt = ops.moe_route(h.to(DEV), wr.to(DEV), None, top, ops.MOE_SCORE_SOFTMAX_ALL, corr.to(DEV), 1.7)
        assert torch.equal(idx.cpu().long().sort(-1).values, chosen.sort(-1).values)
        _close(wgt, torch.gather(s, 1, idx.cpu().long()) * 1.7, torch.float32, "weights")
        gu = (torch.randn(E, 2 * ff, D, generator=g) * 0.2).to(dtype)
        dn = (torch.randn(E, D, ff, generator=g) * 0.2).to(dtype)
        base = torch.randn(T, D, generator=g).to(dtype)
        want = base.double().clone()
        for t in range(T):
            for j in range(top):
                e, w = int(idx[t, j]), float(wgt[t, j])
                if e >= E:
                    want[t] += w * h[t].double()
                else:
                    a = gu[e].double() @ h[t].double()
                    want[t] += w * (dn[e].double() @ (plain.silu(a[:ff]) * a[ff:]))
        y = ops.moe_experts(h.to(DEV), idx, wgt, gu.to(DEV), dn.to(DEV), base=base.to(DEV), identity=ident)
        _close(y, want, dtype, "experts")
    _status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,ps,chunk", [(4, 2, 32, 48, 8, 24), (6, 2, 24, 40, 4, 7), (2, 2, 64, 64, 16, 0), (8, 1, 16, 16, 16, 16)])
def test_norm_store_and_biased_attention_kernels(dtype, H, G, d, dv, ps, chunk):
    """Queries and keys normed over the whole projection, values per head, stored in pages in any order; then every token's
    attention over its request's pages with the distance bias, the chunk and the sink, with one part and with four."""
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(H * 31 + d)
    row = -(-max(d, dv) // 16) * 16
    lens = [37, 1, 90]
    T, pages = sum(lens), 40
    proj = (torch.randn(T, (H + G) * d + G * dv + 8, generator=g)).to(dtype)
    qw, kw = torch.rand(H * d, generator=g) + 0.5, torch.rand(G * d, generator=g) + 0.5
    P = proj.double()
    unit = lambda x: x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5)
    q = (unit(P[:, :H * d]) * qw.double()).view(T, H, d)
    k = (unit(P[:, H * d:(H + G) * d]) * kw.double()).view(T, G, d)
    v = unit(P[:, (H + G) * d:(H + G) * d + G * dv].view(T, G, dv))
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.zeros(3, 24, dtype=torch.int32)
    slots, seg, pos, at = [], [], [], 0
    for s, n in enumerate(lens):
        for b in range(-(-n // ps)):
            table[s, b] = order.pop()
        for i in range(n):
            slots.append(int(table[s, i // ps]) * ps + i % ps)
            seg.append(s)
            pos.append(i)
    slots, seg, pos = (torch.tensor(a, dtype=torch.int32) for a in (slots, seg, pos))
    slopes = torch.tensor([2.0 ** (-8.0 * (a + 1) / H) for a in range(H)])
    want = torch.zeros(T, H, row, dtype=torch.float64)
    cu = [0, lens[0], lens[0] + lens[1]]
    for t in range(T):
        s, i = int(seg[t]), int(pos[t])
        lo = (i // chunk) * chunk if chunk else 0
        for a in range(H):
            kk, vv = k[cu[s] + lo:cu[s] + i + 1, a // (H // G)], v[cu[s] + lo:cu[s] + i + 1, a // (H // G)]
            sc = (kk @ q[t, a]) * 0.3 - float(slopes[a]) * (i - torch.arange(lo, i + 1)).double()
            e = torch.exp(sc)
            want[t, a, :dv] = (e / (1.0 + e.sum())) @ vv
    dev = lambda t: t.to(DEV)
    kp = torch.full((pages, G, ps, row), float("nan"), dtype=dtype, device=DEV)
    vp = torch.full_like(kp, float("nan"))
    qd = ops.whole_norm_store(dev(proj), 0, H * d, (H + G) * d, dev(qw), dev(kw), 1e-5, True, dev(slots), kp, vp, H, G, d, dv, row, ps)
    _close(qd.view(T, H, row)[:, :, :d], q, dtype, "q")
    assert float(qd.view(T, H, row)[:, :, d:].abs().sum()) == 0.0
    for splits in (1, 4):
        out = torch.empty(T, H * row, dtype=dtype, device=DEV)
        scratch = torch.empty(ops.attention_scratch_floats(T, H, row, splits), dtype=torch.float32, device=DEV)
        ops.paged_attention(qd, kp, vp, out, dev(seg), dev(pos), dev(table), H, G, row, ps, None, 0.3, splits, scratch,
                            slopes=dev(slopes.float()), chunk=chunk or None, sinks=torch.zeros(H, device=DEV))
        _close(out.view(T, H, row), want, dtype, f"attention in {splits} parts")
    _status()


@pytest.mark.gpu
@pytest.mark.parametrize("H,G,d,ps,chunk,window", [(4, 2, 64, 16, 100, None), (8, 2, 128, 16, 192, None), (2, 1, 128, 64, 0, None),
                                                   (6, 2, 48, 8, 70, None), (16, 1, 32, 4, 33, 50), (4, 4, 80, 16, 128, None),
                                                   (2, 2, 64, 32, 64, 40), (2, 2, 64, 16, 20, None), (8, 2, 128, 8, 9, None)])
def test_biased_attention_on_tensor_cores(H, G, d, ps, chunk, window):
    """The bfloat16 kernels: portions of prompts (with tensor maps over the pages where the head size has them) beside
    single tokens in one and in four parts, over pages in any order that hold NaN wherever nothing was stored.  Sinks
    differ by head; requests start in the middle of a chunk, cross chunk borders and are longer than one tile of keys."""
    from pico_vllm_b200 import ops
    g = torch.Generator().manual_seed(H * 131 + d + chunk)
    # (keys already cached, tokens the step brings)
    reqs = [(0, 150), (97, 1), (60, 141), (299, 1), (chunk or 77, 2), (max(chunk - 1, 0), 1), (0, 1), (130, 70)]
    total = [a + b for a, b in reqs]
    n_pages = sum(-(-n // ps) for n in total) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(len(reqs), max(-(-n // ps) for n in total) + 1, dtype=torch.int32)
    kp = torch.full((n_pages, G, ps, d), float("nan"), dtype=torch.bfloat16)
    vp = torch.full_like(kp, float("nan"))
    K = [torch.randn(n, G, d, generator=g).to(torch.bfloat16) for n in total]
    V = [torch.randn(n, G, d, generator=g).to(torch.bfloat16) for n in total]
    for s, n in enumerate(total):
        for b in range(-(-n // ps)):
            table[s, b] = order.pop()
            m = min(ps, n - b * ps)
            kp[table[s, b], :, :m] = K[s][b * ps:b * ps + m].transpose(0, 1)
            vp[table[s, b], :, :m] = V[s][b * ps:b * ps + m].transpose(0, 1)
    seg, pos, cu = [], [], [0]
    for s, (a, b) in enumerate(reqs):
        seg += [s] * b
        pos += list(range(a, a + b))
        cu.append(cu[-1] + b)
    T = len(seg)
    q = (torch.randn(T, H * d + 16, generator=g) * 1.5).to(torch.bfloat16)
    slopes = torch.tensor([2.0 ** (-8.0 * (a + 1) / H) for a in range(H)])
    sinks = torch.linspace(-1.0, 2.0, H)
    want = torch.zeros(T, H, d, dtype=torch.float64)
    for t in range(T):
        s, i = seg[t], pos[t]
        lo = (i // chunk) * chunk if chunk else 0
        if window:
            lo = max(lo, i + 1 - window)
        for a in range(H):
            kk, vv = K[s][lo:i + 1, a // (H // G)].double(), V[s][lo:i + 1, a // (H // G)].double()
            sc = (kk @ q[t, a * d:(a + 1) * d].double()) * 0.11 - float(slopes[a]) * (i - torch.arange(lo, i + 1)).double()
            e = torch.exp(sc)
            want[t, a] = (e / (math.exp(float(sinks[a])) + e.sum())) @ vv
    dev = lambda x: x.to(DEV)
    kd, vd = dev(kp), dev(vp)
    pre = [s for s, (a, b) in enumerate(reqs) if b > 1]
    dec = [cu[s] for s, (a, b) in enumerate(reqs) if b == 1]
    for maps in (False, True):
        k2, v2 = (ops.make_kv_tensor_map_2d(kd), ops.make_kv_tensor_map_2d(vd, values=True)) if maps else (None, None)
        if maps and (k2 is None or v2 is None):
            continue
        for splits in (1, 4):
            out = torch.full((T, H * d), float("nan"), dtype=torch.bfloat16, device=DEV)
            scratch = torch.empty(ops.attention_scratch_floats(T, H, d, splits), dtype=torch.float32, device=DEV)
            ops.paged_attention_mma(dev(q), kd, vd, out, dev(torch.tensor(seg, dtype=torch.int32)),
                                    dev(torch.tensor(pos, dtype=torch.int32)), dev(table), dev(torch.tensor(cu, dtype=torch.int32)),
                                    dev(torch.tensor(pre, dtype=torch.int32)), len(pre), max(b for a, b in reqs),
                                    dev(torch.tensor(dec, dtype=torch.int32)), len(dec), H, G, d, ps, window, 0.11, splits, scratch,
                                    None, None, k2, v2, 0, slopes=dev(slopes.float()), chunk=chunk or None, sinks=dev(sinks.float()))
            _close(out.view(T, H, d), want, torch.bfloat16, f"tensor maps {maps}, {splits} parts")
    _status()


# ------------------------------------------------------------------ through the entry points
def _folder(tmp_path, raw, tensors):
    from pico_vllm_b200.registry import config_from_dict
    from safetensors.torch import save_file
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config_from_dict(raw).to_dict()))
    save_file(tensors, str(folder / "model.safetensors"))
    return str(folder)


def test_greedy_generation_through_the_entry_point(tmp_path):
    from pico_vllm_b200 import LLM, SamplingParams
    raw = SHAPES["a"]
    tensors = _tensors(raw, SEEDS["a"])
    llm = LLM(_folder(tmp_path, raw, tensors), dtype="float32", max_cache_tokens=1024, device=DEV)
    prompts = [helpers.random_ids(n, raw["vocab"], 70 + n) for n in (4, 23, 61)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert list(o.token_ids) == _greedy(raw, tensors, p, 12)


def test_command_line_writes_a_model_folder_and_generates(tmp_path, capsys):
    from pico_vllm_b200.cli import main
    from safetensors.torch import load_file
    (tmp_path / "config.json").write_text(json.dumps(SHAPES["d"]))
    folder = str(tmp_path / "model")
    assert main(["random-model", "--config", str(tmp_path / "config.json"), "--seed", "9", "--out", folder, "--std", str(STD)]) == 0
    capsys.readouterr()
    prompts = [[5, 17, 3], [9, 9]]
    rc = main(["run", "--model", folder, "--dtype", "float32", "--prompt-ids", "5,17,3", "--prompt-ids", "9,9",
               "--max-new-tokens", "5", "--temperature", "0", "--num-gpu-blocks", "32", "--ignore-eos"])
    assert rc == 0
    lines = [l for l in capsys.readouterr().out.splitlines() if l.startswith("[")]
    printed = {int(l[1:l.index("]")]): [int(t) for t in l.split("] ")[1].split()] for l in lines}
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    for rid, p in enumerate(prompts):       # prompt and generated tokens are printed together
        assert printed[rid] == p + _greedy(SHAPES["d"], tensors, p, 5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("keep", ["all", "no attention", "attention only"])
def test_trace_replay_of_a_model_folder(tmp_path, dtype, keep):
    """Also models that need no pages at all (no layer with attention) and models whose every layer has both pages and states."""
    raw = _raw("c", dtype)
    if keep != "all":
        raw["layers"] = [l for l in raw["layers"] if (l["type"] == "parallel") == (keep == "attention only")]
    tensors = _tensors(raw, SEEDS["c"])
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 300 + i) for i, n in enumerate([40, 7, 95, 33, 64])}
    steps = helpers.trace_mixed(reqs, max_live=4, seed=1)
    lines = "".join(json.dumps(dict(step=i, **st)) + "\n" for i, st in enumerate(steps))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", _folder(tmp_path, raw, tensors),
                        "--dtype", dtype, "--out", str(out), "--max-tokens", str(helpers.live_token_peak(steps))],
                       input=lines, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    logits = _oracle(raw, tensors, reqs)
    got = [None if w is None else torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, raw["vocab"]))
           for i, w in enumerate(helpers.expected_logits(steps, reqs, logits))]
    _compare(steps, reqs, got, logits, dtype, f"replay ({keep})")
