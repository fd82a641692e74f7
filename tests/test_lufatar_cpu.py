"""CPU side of the Lufatar integration: configuration, registry, layer-run order, and sanity of the
float64 oracle itself (causality, the sink, the convolution's reach, the router's groups)."""
import json

import pytest
import torch

from oracle import lufatar_oracle as O
from tests.test_lufatar_gpu import CONFIGS
from vila_b200.model.lufatar import LufatarConfig, LufatarForCausalLM
from vila_b200.model.registry import LANGUAGE_MODELS, language_model_architecture

F64 = torch.float64


def random_weights(cfg_dict, seed=0):
    g = torch.Generator().manual_seed(seed)
    shapes = LufatarConfig.from_dict(cfg_dict).tensor_shapes()
    return {n: (torch.randn(s, generator=g) * (0.1 if len(s) == 1 else 1.5 / s[-1] ** 0.5)).to(torch.bfloat16)
            for n, s in shapes.items()}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_shapes_and_runs(name):
    d = CONFIGS[name]
    cfg = LufatarConfig.from_dict(d)
    assert cfg.to_dict() == json.loads(json.dumps(d))
    shapes = cfg.tensor_shapes()
    for i, spec in enumerate(d["layers"]):
        assert (f"l{i}.norm2" in shapes) == (spec["mlp"] is not None)
        assert (f"l{i}.side.gate" in shapes) == ("token_side" in d)
    assert ("loop.step" in shapes) == ("loop" in d)
    assert shapes["bigram"] == (d["embedding"]["bigram"]["buckets"] + 1, d["width"])
    assert cfg.runs() == O.layer_runs(d)
    model = LufatarForCausalLM(cfg, "cpu")
    assert len(model.latent_widths()) == len(cfg.runs())
    assert len(model.state_shapes()) == (0 if cfg.taps == 1 else sum(2 if d["layers"][i]["mlp"] else 1 for i, _ in cfg.runs()))


def test_layer_runs_of_a_repeated_block():
    d = json.loads(json.dumps(CONFIGS["odd"]))
    assert O.layer_runs(d) == [(0, -1), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, -1)]
    del d["loop"]
    assert LufatarConfig.from_dict(d).runs() == [(i, -1) for i in range(4)]


def test_bad_configs_are_refused():
    for change in (lambda d: d["layers"][0].update(type="something_else"),
                   lambda d: d["layers"][0]["mixer"].update(kv_heads=2),            # 3 heads over 2 key heads
                   lambda d: d["layers"][0]["mlp"]["router"].update(top=5),         # more than the kept groups hold
                   lambda d: d["norm"].update(groups=5),
                   lambda d: d["loop"].update(stop=9)):
        d = json.loads(json.dumps(CONFIGS["odd"]))
        change(d)
        with pytest.raises(ValueError):
            LufatarConfig.from_dict(d)


def test_registry_names_the_architecture(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CONFIGS["plain"]))
    assert language_model_architecture(tmp_path) == "Lufatar" and LANGUAGE_MODELS["Lufatar"] is LufatarForCausalLM


def test_oracle_is_causal_and_its_sink_counts_once():
    cfg = CONFIGS["odd"]
    w = random_weights(cfg, 1)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(2)).tolist()
    full = O.forward(cfg, w, toks)[0]
    assert float((O.forward(cfg, w, toks[:17])[0] - full[:17]).abs().max()) < 1e-9
    p = O.softmax_plus_one(torch.zeros(1, 3, dtype=F64))
    assert torch.allclose(p, torch.full_like(p, 0.25))      # three keys + the sink share the mass
    p = O.softmax_plus_one(torch.tensor([[-800.0, -801.0]], dtype=F64))
    assert float(p.sum()) < 1e-300 or float(p.sum()) == 0.0  # far below the sink: nearly nothing


def test_oracle_convolution_reach_and_router_groups():
    h = torch.zeros(10, 2, dtype=F64)
    h[4] = 1.0
    w = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 0.0]], dtype=F64)     # taps = 3: weights of t-2, t-1, t
    out = O.short_conv_residual(h, w)
    assert out[:, 0].tolist() == [0, 0, 0, 0, 101.0, 10.0, 1.0, 0, 0, 0] and out[:, 1].tolist() == h[:, 1].tolist()
    # 2 groups of 3, one kept: group 0 has the single best expert, group 1 the best pair
    W = {"r.router": torch.zeros(6, 4, dtype=F64),
         "r.correction": torch.tensor([0.9, 0.0, 0.0, 0.6, 0.5, 0.1], dtype=F64)}
    r = {"experts": 6, "top": 2, "groups": {"count": 2, "keep": 1}}
    idx, wt = O.route(torch.ones(1, 4, dtype=F64), W, "r.", r)
    assert sorted(idx[0].tolist()) == [3, 4] and torch.allclose(wt, torch.full_like(wt, 0.5))
