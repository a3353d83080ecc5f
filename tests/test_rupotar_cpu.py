"""Rupotar without a GPU: configuration, the model as data, the tensor list,
and the plain implementation against its own token-by-token forms."""
import json

import pytest
import torch

import plain_rupotar as plain
import rupotar_tiny as tiny


def parsed(name):
    from foundry_b200.config.rupotar import RupotarConfig
    return RupotarConfig.parse(tiny.CONFIGS[name])


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_config_round_trip_and_registry(name):
    from foundry_b200.config.registry import resolve_architecture
    cfg = parsed(name)
    assert type(cfg).parse(json.dumps(cfg.to_json())) == cfg
    assert resolve_architecture(tiny.CONFIGS[name]).name == "Rupotar"
    assert cfg.width == tiny.CONFIGS[name]["width"] and len(cfg.layers) == len(tiny.CONFIGS[name]["layers"])


def test_config_refusals():
    from foundry_b200.config import errors
    from foundry_b200.config.rupotar import RupotarConfig
    doc = json.loads(json.dumps(tiny.CONFIGS["looped"]))
    doc["layers"][1]["mixer"]["kv_heads"] = 4
    with pytest.raises(errors.HeadRatio):
        RupotarConfig.parse(doc)
    doc = json.loads(json.dumps(tiny.CONFIGS["looped"]))
    doc["layers"][0]["type"] = "hyena"
    with pytest.raises(errors.UnsupportedOption):
        RupotarConfig.parse(doc)
    doc = json.loads(json.dumps(tiny.CONFIGS["looped"]))
    doc["loop"]["stop"] = 9
    with pytest.raises(errors.ConfigJson):
        RupotarConfig.parse(doc)
    doc = json.loads(json.dumps(tiny.CONFIGS["looped"]))
    del doc["norm"]
    with pytest.raises(errors.ConfigJson):
        RupotarConfig.parse(doc)


def test_schedule_of_a_loop_gives_every_pass_its_own_cache():
    from foundry_b200.models.rupotar import build_rupotar_spec
    spec = build_rupotar_spec(parsed("looped"))
    runs = [(e.layer, e.junction) for e in spec.schedule]
    assert runs == [(0, (0, 0)), (1, None), (0, (0, 1)), (1, None), (0, (0, 2)), (1, None),
                    (2, None), (3, None)]
    assert [e.cache for e in spec.schedule] == list(range(8))
    assert runs == [(i, None if t is None else (0, t)) for i, t in plain.run_order(tiny.CONFIGS["looped"])]
    straight = build_rupotar_spec(parsed("straight"))
    assert [(e.layer, e.junction) for e in straight.schedule] == [(0, None), (1, None), (2, None)]
    assert not straight.junctions


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_tensor_list_and_sizes_from_shapes(name):
    """The model lists exactly the tensors of the design, once the ranks that
    only the tensors' shapes give are read from there."""
    from foundry_b200.config.rupotar import complete_from_files
    from foundry_b200.engine.model import expected_tensors
    from foundry_b200.models.rupotar import build_rupotar_spec
    shapes = tiny.tensor_shapes(tiny.CONFIGS[name], *tiny.RANKS[name])

    class Files:
        def __contains__(self, key):
            return key in shapes

        def entry(self, key):
            return type("E", (), {"shape": shapes[key]})
    cfg = complete_from_files(parsed(name), Files())
    ranks = {(l.type, l.decay_rank, l.gate_rank) for l in cfg.layers if l.type != "attention"}
    assert ranks == {("wkv", tiny.RANKS[name][0], None),
                     ("channel_delta", tiny.RANKS[name][0], tiny.RANKS[name][1])}
    listed = expected_tensors(build_rupotar_spec(cfg))
    assert {k: tuple(v.shape) for k, v in listed.items()} == shapes


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_plain_recurrent_mixers_equal_their_stepwise_forms(name):
    cfg, w = tiny.CONFIGS[name], {k: v.double() for k, v in tiny.random_weights(name).items()}
    torch.manual_seed(3)
    h = torch.randn(11, cfg["width"], dtype=torch.float64)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}.mix"
        if layer["type"] == "wkv":
            a = plain.wkv_time_mix(layer["mixer"], w, p, h, cfg["norm"]["eps"])
            b = plain.wkv_stepwise(layer["mixer"], w, p, h, cfg["norm"]["eps"])
        elif layer["type"] == "channel_delta":
            a = plain.gated_delta(layer["mixer"], w, p, h, cfg["norm"]["eps"])
            b = plain.gated_delta_stepwise(layer["mixer"], w, p, h, cfg["norm"]["eps"])
        else:
            continue
        assert float((a - b).abs().max()) < 1e-10 * max(1.0, float(a.abs().max()))


def test_plain_attention_mask_sink_and_bias():
    """One query over three keys by hand: the sink's one in the denominator, the
    bias by the tokens' own distance, the window with a kept first token."""
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0,
         "mask": {"size": 2, "keep_first": 1}}
    eye = torch.eye(2, dtype=torch.float64)
    w = {"a.q": eye, "a.k": eye, "a.v": torch.tensor([[1.0, 0.0]], dtype=torch.float64),
         "a.q.norm": torch.ones(2, dtype=torch.float64), "a.k.norm": torch.ones(2, dtype=torch.float64),
         "a.o": torch.ones(1, 1, dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.0], [2.0, 0.0], [3.0, 0.0], [1.0, 0.0]], dtype=torch.float64)
    out = plain.sink_attention(m, w, "a", h, 1e-12, steep=8.0)
    # after the whole-projection norm every q and k is (sqrt 2, 0); v is h[:, 0]
    slope, s = 2.0 ** -8.0, 2.0
    import math
    # the last query (i = 3) sees j = 3, 2 (window 2) and j = 0 (kept), not j = 1
    e = [math.exp(s - slope * 3), math.exp(s - slope * 1), math.exp(s)]
    want = (e[0] * 1.0 + e[1] * 3.0 + e[2] * 1.0) / (1.0 + sum(e))
    assert abs(float(out[3, 0]) - want) < 1e-12
    assert plain.visible(70, 1, 70, 0) and not plain.visible(70, 0, 70, 0) and plain.visible(70, 0, 70, 1)
