"""The Banazen design through the step function, the cache and the batch building on the CPU, with the kernels replaced by
torch doubles (tests/fake_ops.py): several cache entries per layer (pages beside state slots), latents shared between
layers, positions, cache rows, page and slot reuse and wanted rows, in every way of cutting requests into steps."""
import pytest
import torch

import fake_ops
import helpers
import plain_banazen as plain
from test_banazen_gpu import SHAPES, SEEDS, _tensors


def _runner(raw, tensors, max_tokens, page_size, max_num_seqs=4):
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine import ModelRunner, make_cache, model_from_tensors
    from pico_vllm_b200.registry import config_from_dict
    ecfg = EngineConfig(dtype="float32", page_size=page_size, max_cache_tokens=max_tokens, max_num_seqs=max_num_seqs,
                        use_cuda_graph=False, device="cpu")
    model = model_from_tensors(config_from_dict(raw), tensors, ecfg)
    return ModelRunner(model, make_cache(model, ecfg, poison_freed=True), ecfg)


@pytest.fixture
def on_cpu(monkeypatch):
    fake_ops.install(monkeypatch)
    import pico_vllm_b200.engine.core as core
    monkeypatch.setattr(core, "_require_device", lambda device: None)


@pytest.mark.parametrize("name,page_size", [("a", 8), ("b", 16), ("c", 4)])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_every_cutting_matches_plain(on_cpu, name, page_size, cut):
    raw = SHAPES[name]
    tensors = _tensors(raw, SEEDS[name])
    reqs = {f"r{i}": helpers.random_ids(n, raw["vocab"], 40 + i) for i, n in enumerate([1, 7, 30, 45, 18])}
    steps = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_tail_decode(r, 12),
             "portions": helpers.trace_portions, "mixed": lambda r: helpers.trace_mixed(r, max_live=3, seed=2)}[cut](reqs)
    runner = _runner(raw, tensors, helpers.live_token_peak(steps), page_size, max_num_seqs=3)
    logits = {rid: plain.forward(raw, tensors, ids) for rid, ids in reqs.items()}
    want = helpers.expected_logits(steps, reqs, logits)
    got = helpers.replay(runner, steps)
    for i, (g, w) in enumerate(zip(got, want)):
        assert (g is None) == (w is None)
        if w is not None:
            helpers.assert_close_logits(g, w.float(), 5e-5, f"{name}/{cut} step {i}")
    assert all(g.pool.in_use == 0 for g in runner.cache.groups)


def test_a_slot_taken_again_starts_from_zero_states(on_cpu):
    """The memory and the convolutions' last inputs belong to the request that holds the slot: the next request in the same
    slot starts from zeros, whatever the one before left there."""
    raw = SHAPES["a"]
    tensors = _tensors(raw, SEEDS["a"])
    ids = helpers.random_ids(20, raw["vocab"], 3)
    runner = _runner(raw, tensors, 64, 8, max_num_seqs=1)
    first = helpers.replay(runner, helpers.trace_whole({"x": ids}))[0]
    assert all(float(s.abs().max()) > 0 for s in runner.cache.states.values() if s.numel())      # the slot is left dirty
    again = helpers.replay(runner, helpers.trace_whole({"y": ids}))[0]
    assert torch.equal(first, again)
