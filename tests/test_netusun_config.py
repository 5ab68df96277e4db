"""Reading, refusing and laying out Netusun configurations; runs without a GPU."""

import copy

import pytest

import netusun_cases as cases
import plain_netusun as plain
from stride_b200.config import ConfigError, NetusunConfig, config_from_dict
from stride_b200.engine.loading import _declarations, footprint


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_declarations_are_the_checkpoints_tensors(case):
    cfg = cases.CASES[case]
    state = cases.seeded_state(cfg, 1)
    config = config_from_dict(cfg)
    assert isinstance(config, NetusunConfig)
    declared = _declarations(config)
    assert set(declared) == set(state)
    for name, decl in declared.items():
        assert tuple(decl.shape) == tuple(state[name].shape), name
    assert config_from_dict(config.to_dict()) == config


@pytest.mark.parametrize("case", sorted(cases.CASES))
def test_the_run_order_is_the_plain_one(case):
    cfg = cases.CASES[case]
    spec = config_from_dict(cfg).to_model_spec()
    assert [(e.layer, e.enters_pass) for e in spec.schedule] == plain.run_order(cfg)
    assert [e.cache for e in spec.schedule] == list(range(cases.run_count(cfg)))          # a cache and a state of its own per run
    assert (spec.pass_input is None) == ("loop" not in cfg)


def test_layout_of_a_layer_list():
    spec = config_from_dict(cases.CASE_A).to_model_spec()
    assert [(e.layer, e.enters_pass) for e in spec.schedule] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert spec.pass_input.passes == 3 and spec.pass_input.mix_name == "loop.in" and spec.head_spec().name is None
    assert all(layer.kind == "sandwich" for layer in spec.layers)
    assert dict(spec.layers[1].mixer_out_norm.params) == {"tensor": "l1.norm1b", "scale_tensor": "l1.ls1"}
    assert dict(spec.layers[1].ffn_out_norm.params)["scale_tensor"] == "l1.ls2" and "scale_tensor" not in dict(spec.layers[1].mixer_norm.params)
    assert spec.layers[0].feed_forward is None and spec.layers[0].ffn_norm is None and spec.layers[0].ffn_out_norm is None
    lstm, lat, win = (spec.layers[i].mixer for i in range(3))
    assert lstm.kind == "mlstm" and dict(lstm.params) == {"value_dim": 16, "gate_cap": 6.0, "norm_eps": 1e-6}
    p = dict(lat.params)
    assert lat.kind == "latent_attention" and (p["rot_dim"], p["value_dim"], p["kv_rank"], p["q_rank"]) == (8, 24, 40, 24)
    assert p["output_gate"] == "full" and p["sinks"] is True and p["pairing"] == "halves" and lat.position.scaling is None
    p = dict(win.params)
    assert win.kind == "attention" and win.window == 20 and win.position.kind == "none" and not win.bias
    assert (p["conv"], p["softcap"], p["qk_norm"], p["sinks"], p["value_dim"]) == (4, 5.0, "weighted", "zero", 24)
    routed = dict(spec.layers[2].feed_forward.params)
    assert spec.layers[2].feed_forward.activation == "silu" and routed["router"] == "softmax_groups"
    assert (routed["experts"], routed["top"], routed["groups"], routed["keep"], routed["route_scale"], routed["shared"]) == (8, 2, 4, 2, 2.0, 40)
    assert "shared" not in dict(spec.layers[3].feed_forward.params) and dict(spec.layers[3].feed_forward.params)["groups"] == 1
    yarn = config_from_dict(cases.CASE_C).to_model_spec().layers[0].mixer.position.scaling
    assert (yarn.rope_type, yarn.factor, yarn.original_max_position_embeddings, yarn.high_freq_factor, yarn.low_freq_factor) == ("yarn", 4.0, 64, 8.0, 1.0)


def test_footprint_counts_every_run():
    f = footprint(config_from_dict(cases.CASE_A), "bfloat16")
    # three runs of the latent layer (40 + 8 a token) and of the first windowed layer (2 x 16 keys, 2 x 24 values), one of the second (3 x 8 twice)
    assert f["kv_bytes_per_token"] == 2 * (3 * 48 + 3 * 80 + 48)
    # the matrix LSTM's memory (S, n and m of two heads), the tails of 3 and 1 projected rows of the windowed layers' runs
    assert f["state_bytes_per_request"] == 4 * ((2 * 24 * 16 + 2 * 24 + 2) + 3 * 3 * (4 * 16 + 2 * 16 + 2 * 24) + 1 * (3 * 8 * 3))


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="wkv"), "type"),
    (lambda d: d["layers"][2]["mixer"].update(kv_heads=3), "group"),
    (lambda d: d["layers"][2]["mixer"].update(dim=300), "256"),
    (lambda d: d["layers"][2]["mixer"].update(conv=17), "taps"),
    (lambda d: d["layers"][2]["mixer"].update(softcap=0.0), "softcap"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda d: d["layers"][0]["mixer"].update(gate_cap=0.0), "gate_cap"),
    (lambda d: d["layers"][1]["mlp"].update(kind="conv"), "kind"),
    (lambda d: d["layers"][2]["mlp"]["router"].update(top=5), "choices"),
    (lambda d: d["loop"].update(stop=1), "enclose"),
    (lambda d: d["loop"].update(stop=9), "enclose"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_refusals(change, message):
    d = copy.deepcopy(cases.CASE_A)
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)
