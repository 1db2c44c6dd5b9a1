"""The Banazen configuration reader, the builder's tensor names and cache layout, and the random-weights folder (CPU)."""
import copy
import json

import pytest
import torch

from test_banazen_gpu import SHAPES, _tensors


def _cfg(raw):
    from pico_vllm_b200.registry import config_from_dict
    return config_from_dict(raw)


@pytest.mark.parametrize("name", sorted(SHAPES))
def test_reads_back_what_it_writes(name):
    cfg = _cfg(SHAPES[name])
    assert cfg.architecture == "Banazen" and _cfg(cfg.to_dict()) == cfg
    assert _cfg(json.loads(json.dumps(cfg.to_dict()))) == cfg


def test_absent_keys_have_the_documented_meaning():
    raw = copy.deepcopy(SHAPES["b"])
    del raw["embedding"], raw["logit_scale"]
    cfg = _cfg(raw)
    assert cfg.embedding_scale == 1.0 and cfg.logit_scale == 1.0 and cfg.side_dim is None
    assert cfg.layers[0].mixer.window is None and cfg.layers[2].mixer.window == 16
    raw["layers"][1]["mixer"]["right"].pop("decay_rank")
    assert _cfg(raw).layers[1].mixer.right.decay_rank is None


@pytest.mark.parametrize("change,word", [
    (lambda r: r["layers"][2]["mixer"].update(kv_from=3), "kv_from"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda r: r["layers"][2]["mixer"].update(kv_rank=32), "kv_rank"),
    (lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=15), "dims"),
    (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda r: r["layers"][1].update(type="mamba2"), "type"),
    (lambda r: r["layers"][0]["mlp"].update(kind="other"), "kind"),
    (lambda r: r.pop("vocab"), "vocab"),
])
def test_errors_name_the_key(change, word):
    from pico_vllm_b200.errors import ConfigError
    raw = copy.deepcopy(SHAPES["a"])
    change(raw)
    with pytest.raises(ConfigError) as e:
        _cfg(raw)
    assert word in str(e.value)


def test_tensor_names_cache_entries_and_sizes_the_tensors_give():
    from pico_vllm_b200.errors import WeightError
    from pico_vllm_b200.parts import FixedState, PagedKV, PagedLatent
    from pico_vllm_b200.registry import build_model
    from pico_vllm_b200.weights.loader import check_tensors, wanted_tensors
    raw = SHAPES["a"]
    model = build_model(_cfg(raw))
    want = wanted_tensors(model)
    for n in ("embed", "side.embed", "l0.norm1", "l0.mix.left.q.conv", "l0.mix.left.out", "l0.mix.right.a2", "l0.mix.right.A_log",
              "l0.mlp.gate", "l1.mix.dkv.norm", "l1.mlp.correction", "l1.mlp.e5.down", "l1.mlp.shared.sg", "l1.side.proj",
              "l3.side.norm", "final.norm", "head"):
        assert n in want, n
    assert "l2.mix.dkv" not in want and "l2.mlp.gate" not in want          # reads layer 1's latents; has no feed-forward
    assert want["side.embed"] == (211, 4 * 10) and want["l0.mix.right.a1"] == (6, 96) and want["l1.mlp.shared.sg"] == (1, 96)
    kinds = [type(e) for e in model.cache_entries]
    assert kinds == [PagedKV, FixedState, FixedState, FixedState, PagedLatent, PagedKV, FixedState, FixedState, FixedState]
    assert model.cache_entries[4] == PagedLatent(48, 24)                   # a latent of 40 in a row of 48, the window of layer 1
    assert model.order[2].cache == 4 and model.order[2].store is False
    # without the two inner sizes in the configuration, whatever the tensors have is taken
    loose = copy.deepcopy(raw)
    for k in ("decay_rank", "gate_rank"):
        loose["layers"][0]["mixer"]["right"].pop(k)
    tensors = _tensors(raw, 1)
    model = build_model(_cfg(loose))
    check_tensors(model, {n: tuple(t.shape) for n, t in tensors.items()}, "test")
    bad = {n: tuple(t.shape) for n, t in tensors.items()}
    bad["l0.mix.right.q"] = (7, 96)
    del bad["l3.side.gate"]
    with pytest.raises(WeightError) as e:
        check_tensors(model, bad, "test")
    assert e.value.missing == ["l3.side.gate"] and e.value.wrong_shape == ["l0.mix.right.q"]


def test_random_weights_need_the_sizes_the_tensors_would_give():
    from pico_vllm_b200.errors import ConfigError
    from pico_vllm_b200.weights import random_tensors
    raw = copy.deepcopy(SHAPES["a"])
    raw["layers"][0]["mixer"]["right"].pop("gate_rank")
    with pytest.raises(ConfigError) as e:
        random_tensors(_cfg(raw), 1)
    assert "l0.mix.right.g1" in str(e.value)


def test_random_weights_folder(tmp_path):
    from pico_vllm_b200.config.base import read_config_json
    from pico_vllm_b200.weights import write_random_model
    from safetensors.torch import load_file
    cfg = _cfg(SHAPES["c"])
    folder = write_random_model(cfg, 3, str(tmp_path / "m"))
    assert _cfg(read_config_json(folder)) == cfg
    t = load_file(folder + "/model.safetensors")
    assert t["l1.mix.right.g2"].shape == (4 * 12, 7) and t["l0.mix.uk"].dtype == torch.bfloat16
