"""Reading, refusing and laying out Tutizen configurations; runs without a GPU."""

import copy

import pytest

import tutizen_cases as cases
from stride_b200.config import ConfigError, TutizenConfig, config_from_dict
from stride_b200.engine.loading import _declarations, footprint


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_declarations_are_the_checkpoints_tensors(case):
    cfg = cases.CASES[case]
    state = cases.seeded_state(cfg, 1)
    config = config_from_dict(cfg)
    assert isinstance(config, TutizenConfig)
    declared = _declarations(config)
    assert set(declared) == set(state)
    for name, decl in declared.items():
        assert tuple(decl.shape) == tuple(state[name].shape), name
    assert config_from_dict(config.to_dict()) == config


def test_layout_of_a_layer_list():
    spec = config_from_dict(cases.CASE_A).to_model_spec()
    assert [(e.layer, e.cache, e.writes_cache) for e in spec.schedule] == [(0, 0, True), (1, 0, False), (2, 2, True), (3, 2, False)]
    assert all(layer.kind == "output_norm" and layer.residual_mult == 0.7 for layer in spec.layers)
    first, second, third = (dict(spec.layers[i].mixer.params) for i in range(3))
    assert first["qk_norm"] == first["v_norm"] == "unit" and first["distance_slopes"] == 8.0 and first["output_gate"] == "head"
    assert "borrowed_kv" not in first and second["borrowed_kv"] is True and third["value_dim"] == 24
    assert spec.layers[0].mixer.position.kind == "none" and spec.layers[0].mixer.bias
    assert dict(spec.layers[0].mixer_norm.params)["shape"] == "scalar"
    assert spec.layers[2].feed_forward is None and spec.layers[2].ffn_norm is None
    ff = spec.layers[0].feed_forward
    assert ff.kind == "swiglu" and ff.activation == "swish_clamped" and dict(ff.params)["limit"] == 1.0 and dict(ff.params)["alpha"] == 1.702
    routed = dict(spec.layers[1].feed_forward.params)
    assert (routed["experts"], routed["top"], routed["groups"], routed["keep"], routed["route_scale"]) == (8, 2, 4, 2, 2.5)
    assert routed["shared"] == 40 and routed["shared_limit"] == 0.8 and routed["shared_gate"] and routed["limit"] == 1.2
    plain_router = dict(spec.layers[3].feed_forward.params)
    assert (plain_router["groups"], plain_router["keep"]) == (1, 1) and "shared" not in plain_router
    assert dict(spec.embedding_spec().params)["sinusoid"] == 10000.0 and spec.head_spec().name == "head"


def test_footprint_counts_only_the_layers_that_keep_pages():
    f = footprint(config_from_dict(cases.CASE_A), "bfloat16")
    # layer 0 keeps keys and values of 1 x 32, layer 2 keys of 4 x 16 and values of 4 x 24; the borrowing layers keep nothing
    assert f["kv_bytes_per_token"] == 2 * (2 * 32 + 4 * 16 + 4 * 24) and f["state_bytes_per_request"] == 0


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="wkv"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=2), "group"),
    (lambda d: d["layers"][0]["mixer"].update(dim=300), "256"),
    (lambda d: d["layers"][1]["mixer"].update(kv_from=1), "earlier"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "of its own"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=0), "must equal"),
    (lambda d: d["layers"][0]["mlp"].update(limit=0.0), "limit"),
    (lambda d: d["layers"][0]["mlp"].update(kind="conv"), "kind"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=5), "choices"),
    (lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda d: d["layers"][1]["mlp"].pop("router"), "router"),
    (lambda d: d.pop("residual_mult"), "residual_mult"),
    (lambda d: d.update(vocab=0), "vocab"),
])
def test_what_is_refused(change, message):
    d = copy.deepcopy(cases.CASE_A)
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_parts_refuse_what_they_cannot_do():
    import torch

    from stride_b200.config import FeedForwardSpec, LayerSpec, MixerSpec, NormSpec, PositionSpec
    from stride_b200.parts import Runtime, build_part
    rt = Runtime("meta", torch.float32, 1, 1)
    norm = NormSpec("rmsnorm", 32, 1e-6, "n.")
    biased = MixerSpec("attention", 32, 2, 1, 16, 0.25, position=PositionSpec("none"), prefix="m.", params=(("output_bias", True),))
    with pytest.raises(ValueError, match="output bias"):         # only the arrangement that norms the output adds it
        build_part("layer", LayerSpec("pre_norm", biased, None, norm, None), rt)
    build_part("layer", LayerSpec("output_norm", biased, None, norm, None), rt)
    with pytest.raises(ValueError, match="limit"):
        build_part("feed_forward", FeedForwardSpec("swiglu", 32, 64, "swish_clamped", "f."), rt)
    with pytest.raises(ValueError, match="groups"):
        build_part("feed_forward", FeedForwardSpec("routed_experts", 32, 8, "swish_clamped", "f.", params=(
            ("experts", 6), ("top", 2), ("router", "sigmoid_groups"), ("groups", 4), ("keep", 1), ("limit", 1.0))), rt)
