"""The Zazilix configuration reader and model builder on the CPU: what config.json keys mean, what is refused and in which
words, which tensors and cache entries the built model asks for, and the plain implementation against itself."""
import copy

import pytest
import torch

import plain_zazilix as plain
from test_zazilix_gpu import SHAPES, SEEDS, _tensors

from pico_vllm_b200.errors import ConfigError
from pico_vllm_b200.parts import FixedState, PagedKV
from pico_vllm_b200.registry import build_model, config_from_dict
from pico_vllm_b200.weights.loader import check_tensors, wanted_tensors


@pytest.mark.parametrize("name", sorted(SHAPES))
def test_round_trip_and_tensor_names(name):
    cfg = config_from_dict(SHAPES[name])
    assert cfg.architecture == "Zazilix" and config_from_dict(cfg.to_dict()) == cfg
    model = build_model(cfg)
    tensors = _tensors(SHAPES[name], SEEDS[name])
    check_tensors(model, {n: tuple(t.shape) for n, t in tensors.items()}, name)
    want = wanted_tensors(model)
    assert want["l0.norm1"] == () and want["final.norm"] == () and want["pos"] == (cfg.max_positions, cfg.width)
    streams = SHAPES[name].get("streams")
    assert ("l0.hc1.mix" in want) == bool(streams)
    if streams:
        assert want["l0.hc1.mix"] == (streams, streams) and want["l0.hc1.in"] == (streams,)
    for i, layer in enumerate(SHAPES[name]["layers"]):
        assert (f"l{i}.norm2" in want) == (layer["mlp"] is not None)
        if layer["mlp"]:
            r = layer["mlp"]["router"]
            assert want[f"l{i}.mlp.router"] == (r["experts"] + r["identity"], cfg.width)
            assert want[f"l{i}.mlp.correction"] == (r["experts"] + r["identity"],)
            assert (f"l{i}.mlp.shared.gate" in want) == ("shared" in layer["mlp"])
            assert f"l{i}.mlp.e{r['experts']}.gate" not in want


def test_cache_entries_of_every_mixer():
    model = build_model(config_from_dict(SHAPES["a"]))
    specs = model.cache_entries
    # parallel: pages of 2 heads padded to 48, and a state [3, 24, 16]; memory: [3, 25, 16] with the normaliser, and the
    # running maximum [3]; state space: [4, 16, 16] and the convolution's last 2 inputs over 64 + 2 * 2 * 16 channels
    assert specs == [PagedKV(2, 48, None), FixedState((3, 24, 16)), FixedState((3, 25, 16)), FixedState((3,)),
                     FixedState((4, 16, 16)), FixedState((2, 128))]
    assert [c.cache for c in model.order] == [(0, 1), (2, 3), (4, 5)]
    one_tap = build_model(config_from_dict(SHAPES["d"]))
    assert one_tap.cache_entries[1] == FixedState((0, 2 * 6 + 2 * 2 * 10))
    assert build_model(config_from_dict(SHAPES["b"])).streams is None


def test_absent_keys_and_refusals():
    raw = copy.deepcopy(SHAPES["b"])
    del raw["embedding"]
    del raw["layers"][0]["mlp"]["router"]["identity"], raw["layers"][0]["mlp"]["router"]["scale"]
    cfg = config_from_dict(raw)
    assert cfg.embedding_scale == 1.0 and cfg.layers[0].mlp.identity == 0 and cfg.layers[0].mlp.scale == 1.0
    assert cfg.layers[2].mixer.left.chunk is None and cfg.streams is None and cfg.max_position_embeddings == 1024
    for change, words in [(lambda r: r["layers"][0].update(type="attention"), "not a mixer of Zazilix"),
                          (lambda r: r.update(streams=9), "'streams' 9 above 8"),
                          (lambda r: r.pop("max_positions"), "'max_positions' is missing"),
                          (lambda r: r["layers"][2]["mixer"]["left"].update(heads=3), "multiple of 'kv_heads'"),
                          (lambda r: r["layers"][0]["mixer"].update(groups=3), "multiple of 'groups'"),
                          (lambda r: r["layers"][0]["mixer"].update(norm_groups=5), "multiple of 'norm_groups'"),
                          (lambda r: r["layers"][1]["mlp"]["router"].update(top=9), "exceeds the 6 router outputs"),
                          (lambda r: r["layers"][1]["mlp"].update(kind="dense"), "not a feed-forward of Zazilix"),
                          (lambda r: r["layers"][1]["mixer"].update(gate_cap=0), "'gate_cap' must be > 0")]:
        bad = copy.deepcopy(SHAPES["b"])
        change(bad)
        with pytest.raises(ConfigError, match=words):
            config_from_dict(bad)


def test_plain_implementation_is_causal_and_its_chunks_are_counted_from_the_start():
    """The oracle itself: logits at a position do not depend on later tokens; a query at the first position of a chunk sees
    only itself and the sink."""
    raw = SHAPES["a"]
    tensors = _tensors(raw, SEEDS["a"])
    ids = list(range(3, 60))
    full = plain.forward(raw, tensors, ids)
    assert torch.allclose(plain.forward(raw, tensors, ids[:30]), full[:30], atol=1e-9)
    m = raw["layers"][0]["mixer"]["left"]
    w = {k[len("l0.mix.left."):]: t.double() for k, t in tensors.items() if k.startswith("l0.mix.left.")}
    h = torch.randn(50, raw["width"], dtype=torch.float64)
    out = plain.chunk_sink_attention(h, w, m, 1e-5)
    h2 = h.clone()
    h2[:24] = torch.randn(24, raw["width"], dtype=torch.float64)           # another first chunk
    assert torch.allclose(plain.chunk_sink_attention(h2, w, m, 1e-5)[24:], out[24:], atol=1e-12)
