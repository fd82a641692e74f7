"""CPU side of the Moronex integration: configuration, checkpoint reader, registry, the host-side
bookkeeping of the token engine's allocators, and sanity of the float64 oracle itself."""
import json

import pytest
import torch

from oracle import moronex_oracle as O
from tests.test_moronex_gpu import CONFIGS
from vila_b200.model.moronex import MoronexConfig, MoronexForCausalLM, read_safetensors
from vila_b200.model.registry import LANGUAGE_MODELS, language_model_architecture
from vila_b200.serving import PageAllocator


def random_weights(cfg_dict, seed=0):
    g = torch.Generator().manual_seed(seed)
    shapes = MoronexConfig.from_dict(cfg_dict).tensor_shapes()
    return {n: (torch.randn(s, generator=g) * (0.1 if len(s) == 1 else 1.5 / s[-1] ** 0.5)).to(torch.bfloat16)
            for n, s in shapes.items()}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_and_shapes(name):
    d = CONFIGS[name]
    cfg = MoronexConfig.from_dict(d)
    assert cfg.to_dict() == json.loads(json.dumps(d))
    shapes = cfg.tensor_shapes()
    for i, spec in enumerate(d["layers"]):
        has_own = spec["type"] == "latent_attention" and "kv_from" not in spec["mixer"]
        assert (f"l{i}.mix.dkv" in shapes) == has_own
        assert (f"l{i}.norm2" in shapes) == (spec["mlp"] is not None)
    assert shapes["head"] == (d["vocab"], d["width"])


def test_bad_configs_are_refused():
    d = json.loads(json.dumps(CONFIGS["odd"]))
    d["layers"][2]["mixer"]["kv_from"] = 0          # layer 0 is recurrent: it has no latent
    with pytest.raises(ValueError):
        MoronexForCausalLM(MoronexConfig.from_dict(d), "cpu")
    d = json.loads(json.dumps(CONFIGS["odd"]))
    d["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        MoronexConfig.from_dict(d)


def test_safetensors_reader_and_registry(tmp_path):
    from safetensors.torch import save_file
    w = random_weights(CONFIGS["narrow"])
    w["table"] = torch.arange(6, dtype=torch.int32).view(2, 3)
    save_file(w, str(tmp_path / "model.safetensors"))
    back = read_safetensors(tmp_path / "model.safetensors")
    assert set(back) == set(w) and all(torch.equal(back[k], w[k]) for k in w)
    assert language_model_architecture(tmp_path) is None
    (tmp_path / "config.json").write_text(json.dumps(CONFIGS["narrow"]))
    assert language_model_architecture(tmp_path) == "Moronex" and "Moronex" in LANGUAGE_MODELS
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llava_llama"}))
    assert language_model_architecture(tmp_path) is None


def test_page_allocator_reuses_released_pages():
    a = PageAllocator(6)
    first = a.alloc(4)
    with pytest.raises(MemoryError):
        a.alloc(3)
    a.release(first[:2])
    again = a.alloc(4)
    assert set(again) & set(first[:2]) == set(first[:2]) and a.available == 0


def test_oracle_is_causal_and_its_sink_counts_once():
    cfg = CONFIGS["odd"]
    w = random_weights(cfg, 1)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(2)).tolist()
    full = O.forward(cfg, w, toks)[0]
    assert float((O.forward(cfg, w, toks[:17])[0] - full[:17]).abs().max()) < 1e-9
    s = torch.zeros(1, 1, 3, dtype=torch.float64)
    p = O.softmax_with_sink(s, torch.zeros(1, dtype=torch.float64))
    assert torch.allclose(p, torch.full_like(p, 0.25))      # three keys + the sink share the mass
