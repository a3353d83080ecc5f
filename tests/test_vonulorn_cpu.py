"""Vonulorn without a GPU: the plain implementation against its own token-by-token
forms, and the configuration, registry and tensor list of the library."""
import math

import pytest
import torch

import plain_vonulorn as plain
import vonulorn_tiny as tiny

F = torch.float64


def double(weights):
    return {k: v.double() for k, v in weights.items()}


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_whole_sequence_mixers_equal_their_stepwise_forms(name):
    cfg = tiny.CONFIGS[name]
    w = double(tiny.random_weights(name))
    gen = torch.Generator().manual_seed(3)
    h = torch.randn(23, cfg["width"], generator=gen, dtype=F)
    for i, layer in enumerate(cfg["layers"]):
        p, m, eps = f"l{i}.mix", layer["mixer"], cfg["norm"]["eps"]
        if layer["type"] == "delta":
            assert torch.allclose(plain.delta_mixer(m, w, p, h, eps),
                                  plain.delta_mixer_stepwise(m, w, p, h, eps), atol=1e-10)
        elif layer["type"] == "latent_attention":
            assert torch.allclose(plain.latent_attention(m, w, p, h, eps),
                                  plain.latent_attention_stepwise(m, w, p, h, eps), atol=1e-10)


def test_rotation_turns_neighbouring_pairs_and_leaves_the_rest():
    x = torch.arange(1, 13, dtype=F).view(1, 12).repeat(2, 1)
    y = plain.rotate_pairs(x, [0, 5], 100.0, 4)
    assert torch.equal(y[0], x[0])                      # position 0 turns nothing
    assert torch.equal(y[1, 4:], x[1, 4:])              # elements beyond `dims` stay
    for i in range(2):
        a = 5 * 100.0 ** (-2 * i / 4)
        u, v = x[1, 2 * i], x[1, 2 * i + 1]
        assert math.isclose(float(y[1, 2 * i]), float(u * math.cos(a) - v * math.sin(a)))
        assert math.isclose(float(y[1, 2 * i + 1]), float(v * math.cos(a) + u * math.sin(a)))


def test_query_temperature_steps_with_the_position():
    t = plain.query_temperature(range(15), 0.5, 7)
    assert float(t[5]) == 1.0 and math.isclose(float(t[6]), 1 + 0.5 * math.log(2))   # (6 + 1) / 7 = 1
    assert math.isclose(float(t[12]), float(t[6])) and math.isclose(float(t[13]), 1 + 0.5 * math.log(3))


def test_sink_takes_its_share_and_has_no_value():
    """One token: the only key's weight is exp(s) / (exp(s) + exp(sink))."""
    m = tiny.CONFIGS["other"]["layers"][1]["mixer"]
    w = double(tiny.random_mixer("latent_attention", m, 64))
    h = torch.randn(1, 64, generator=torch.Generator().manual_seed(1), dtype=F)
    with_sink = plain.latent_attention(m, w, "a", h, 1e-6)
    w["a.sink"] = torch.full_like(w["a.sink"], -1e9)
    without = plain.latent_attention(m, w, "a", h, 1e-6)
    ratio = float((with_sink.norm() / without.norm()))
    assert 0.0 < ratio < 0.999


def test_configuration_registry_and_tensor_list():
    from foundry_b200.config.registry import resolve_architecture
    from foundry_b200.config.vonulorn import VonulornConfig
    from foundry_b200.engine.model import expected_tensors
    from foundry_b200.config import errors
    for name, doc in tiny.CONFIGS.items():
        arch = resolve_architecture(doc)
        assert arch.name == "Vonulorn"
        cfg = arch.parse_config(doc)
        assert isinstance(cfg, VonulornConfig) and cfg.to_json() == doc
        spec = arch.build_spec(cfg)
        want = tiny.tensor_shapes(doc)
        got = {k: tuple(v.shape) for k, v in expected_tensors(spec).items()}
        assert got == want
        kinds = [layer.mixer.kind for layer in spec.layers]
        assert kinds == [{"delta": "gated_delta", "attention": "differential_attention",
                          "latent_attention": "latent_attention"}[l["type"]] for l in doc["layers"]]
        assert all(layer.block.params["residual_scale"] == doc["residual_mult"] for layer in spec.layers)
    bad = {**tiny.CONFIGS["other"], "layers": [{"type": "conv", "mixer": {}, "mlp": None}]}
    with pytest.raises(errors.UnsupportedOption):
        VonulornConfig.parse(bad)
    odd = {**tiny.CONFIGS["other"]}
    odd["layers"] = [dict(odd["layers"][0], mixer=dict(odd["layers"][0]["mixer"], heads=3))]
    with pytest.raises(errors.HeadRatio):
        VonulornConfig.parse(odd)


def test_cache_requests_of_the_three_mixers():
    """Keys of two maps side by side with values of their own; latent rows with no
    value storage; a state row for the delta rule with its convolution tail."""
    from foundry_b200.cache.store import KVRequest, StateRequest
    from foundry_b200.config.registry import resolve_architecture
    from foundry_b200.engine.model import Model
    doc = tiny.CONFIGS["mixed"]
    arch = resolve_architecture(doc)
    model = Model(arch.build_spec(arch.parse_config(doc)), torch.float32, torch.device("meta"))
    req = model.cache_requests()
    assert req[0] == KVRequest(1, 48, None, 0)
    assert req[2] == KVRequest(2, 24, None, 20)
    channels = 2 * 4 * 16 + 4 * 24
    assert req[1] == StateRequest((3 * channels + 4 * 16 * 24,), torch.float32)
