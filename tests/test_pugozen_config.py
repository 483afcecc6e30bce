"""Pugozen on the CPU: the typed configuration, the model's tensors, caches and schedule, and the plain implementation's
own consistency (its recurrences, its sink and its causal mask, which the GPU tests then lean on)."""
import json

import pytest
import torch

import plain_pugozen as plain
from pugozen_cases import CASES, config, delta, pair, retention, shared, write_model


def build(raw, max_positions=256):
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.registry import resolve_architecture
    arch = resolve_architecture(raw)
    cfg = arch.parse_config(dict(raw))
    return cfg, arch.build_model(cfg, max_positions)


def test_config_round_trip_registry_and_schedule():
    from carbon_engine_b200.config.pugozen import PugozenConfig
    from carbon_engine_b200.parts.model import LayerCall
    for name, raw in CASES.items():
        cfg, model = build(raw)
        assert isinstance(cfg, PugozenConfig) and cfg.architecture == "Pugozen"
        assert PugozenConfig.from_dict(json.loads(json.dumps(cfg.to_json_dict()))) == cfg, name
        owners = [l for l in raw["layers"] if l.get("weights_of") is None]
        assert len(model.blocks) == len(owners) and len(model.schedule) == len(raw["layers"])
    _, model = build(CASES["A"])
    assert model.schedule[4:] == [LayerCall(0, 4, True), LayerCall(1, 5, True), LayerCall(2, 6, True)]
    _, model = build(CASES["B"])            # layer 1 runs the weights of layer 3, which comes later
    assert [c.block for c in model.schedule] == [0, 2, 1, 2] and [c.cache for c in model.schedule] == [0, 1, 2, 3]


@pytest.mark.parametrize("bad, text", [
    (lambda r: r["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda r: r["layers"][2]["mixer"].update(decay=[0.9, 0.8]), "one number per head"),
    (lambda r: r["layers"][1]["mixer"]["left"].update(vdim=20), "projected keys"),
    (lambda r: r["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda r: r["layers"][1]["mixer"]["right"].update(conv=0), "conv"),
    (lambda r: r.update(norm={"eps": 0.0}), "positive"),
    (lambda r: r["layers"][0]["mlp"].update(kind="experts"), "mlp"),
    (lambda r: r["layers"][4].update(weights_of=9), "weights_of"),
])
def test_config_errors_name_the_key(bad, text):
    from carbon_engine_b200.config.base import ConfigError
    from carbon_engine_b200.config.pugozen import PugozenConfig
    raw = json.loads(json.dumps(CASES["A"]))
    bad(raw)
    with pytest.raises(ConfigError, match=text):
        PugozenConfig.from_dict(raw)


def test_key_heads_left_out_are_as_many_as_heads():
    raw = json.loads(json.dumps(CASES["C"]))
    del raw["layers"][1]["mixer"]["kv_heads"]
    cfg, model = build(raw)
    assert cfg.layers[1]["mixer"]["kv_heads"] == 3 and model.blocks[1].mixer.kv_heads == 3 and "kv_heads" not in raw["layers"][1]["mixer"]


def test_tensors_and_caches():
    from carbon_engine_b200.parts.base import BundleCacheSpec, PagedCacheSpec, StateCacheSpec
    cfg, model = build(CASES["A"])
    names = {s.name: s.shape for s in model.all_tensor_specs()}
    assert names["l0.mix.q.conv"] == (16, 4) and names["l0.mix.v.conv"] == (48, 4) and names["l0.mix.a"] == (4, 40)
    assert names["l0.mix.dt_bias"] == (4,) and names["l0.mix.g"] == (48, 40) and names["l0.mix.norm"] == (12,)
    assert names["l1.mix.left.k"] == (32, 40) and "l1.mix.left.v" not in names and names["l1.mix.left.q.norm"] == (16,)
    assert names["l1.mix.left.temp"] == (4,) and names["l1.mix.left.sink"] == (4,) and names["l1.mix.left.o"] == (40, 64)
    assert names["l1.mix.right.a2"] == (16, 5) and names["l1.mix.right.dt_bias"] == (16,) and names["l1.mix.right.g2"] == (24, 3)
    assert names["l2.mix.q"] == (36, 40) and names["l2.mix.g"] == (24, 40) and "l2.mlp.up" not in names
    assert names["l3.mlp.up"] == (28, 40) and not any(n.startswith(("l4.", "l5.", "l6.")) for n in names)
    layout = dict(model.cache_layout())
    assert isinstance(layout[0], BundleCacheSpec) and layout[0].main == StateCacheSpec((4, 8, 12), torch.float32)
    assert layout[4] == layout[0] and layout[5] == layout[1] and layout[6] == layout[2] == StateCacheSpec((3, 12, 8), torch.float32)
    assert layout[1].main == PagedCacheSpec(2, 16, 0, None, v_heads=2, v_head_dim=16)
    assert dict(layout[1].extra) == {"1.state": StateCacheSpec((2, 8, 12), torch.float32),
                                     "1.conv": StateCacheSpec((2, 2 * 8 + 2 * 12), torch.float32)}
    # the pair's weights are its members' scales
    pair_mixer = model.blocks[1].mixer
    assert [m.out_scale for m in pair_mixer.members] == [0.7, 0.6] and model.graph_safe
    # ranks left to the checkpoint
    raw = json.loads(json.dumps(CASES["C"]))
    for k in ("a_rank", "g_rank"):
        del raw["layers"][2]["mixer"]["right"][k]
    _, model = build(raw)
    assert {s.name: s.shape for s in model.all_tensor_specs()}["l2.mix.right.a1"] == (-1, 48)


def test_random_model_folder_is_read_back_by_name(tmp_path):
    from carbon_engine_b200.weights.loader import check_tensors
    from carbon_engine_b200.weights.safetensors_io import TensorDirectory
    folder = write_model(CASES["A"], str(tmp_path / "A"))
    cfg, model = build(json.load(open(f"{folder}/config.json")))
    check_tensors(model.all_tensor_specs(), TensorDirectory(folder), model.all_ignorable_tensors())
    cfg2, w = plain.read_model(folder)
    assert cfg2["layers"][5]["weights_of"] == 1 and "l5.norm1" not in w and w["l1.mix.right.a2"].shape == (16, 5)


def test_sketch_config_shares_weights_on_request():
    from carbon_engine_b200.config.pugozen import sketch_config
    cfg = sketch_config(200, 64, 8, 4, 2, 16, 128, shared_from=4)
    assert [l["type"] for l in cfg.layers] == ["delta", "parallel", "parallel", "retention"] * 2
    assert [l.get("weights_of") for l in cfg.layers] == [None] * 4 + [0, 1, 2, 3]
    _, model = build(cfg.to_json_dict())
    assert len(model.blocks) == 4 and len(model.schedule) == 8


# ---- the plain implementation against hand-computed rows ------------------------------------------------------------
def test_plain_recurrences_by_hand():
    F = plain.F
    q = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=F)
    k = torch.tensor([[1.0, 0.0], [0.0, 2.0], [1.0, 0.0]], dtype=F)
    v = torch.tensor([[3.0], [5.0], [7.0]], dtype=F)
    # retention: S0 = k0 v0; S1 = .5 S0 + k1 v1; S2 = .5 S1 + k2 v2
    out = plain.retention_walk(q, k, v, 0.5)
    assert out[:, 0].tolist() == [3.0, 10.0, 0.25 * 3 + 7 + 0.5 * 10]
    # delta rule, decay 1, beta 1: a key written twice is overwritten, not added
    g, beta = torch.ones(3, 2, dtype=F), torch.ones(3, dtype=F)
    out = plain.delta_rule_walk(q, torch.tensor([[1.0, 0.0]] * 3, dtype=F), v, g, beta)
    assert out[:, 0].tolist() == [3.0, 0.0, 7.0]
    # a decay per key channel acts on the rows of S
    g2 = torch.tensor([[1.0, 1.0], [0.5, 1.0], [1.0, 1.0]], dtype=F)
    out = plain.delta_rule_walk(torch.tensor([[1.0, 0.0]] * 3, dtype=F), torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.0, 1.0]], dtype=F), v, g2, beta)
    assert out[:, 0].tolist() == [3.0, 1.5, 1.5]


def test_plain_attention_sink_mask_and_convolution_by_hand():
    F = plain.F
    q = torch.zeros(3, 1, 2, dtype=F)                   # all scores 0: weights are equal
    k = torch.zeros(3, 1, 2, dtype=F)
    v = torch.tensor([[[2.0]], [[4.0]], [[12.0]]], dtype=F)
    out = plain.sink_softmax_attention(q, k, v, 1.0, torch.ones(1, dtype=F), torch.zeros(1, dtype=F))
    # the sink (exp 0 = 1) counts once in every denominator and brings no value; a query sees itself and what came before
    assert torch.allclose(out[:, 0, 0], torch.tensor([2 / 2, 6 / 3, 18 / 4], dtype=F))
    out = plain.sink_softmax_attention(q, k, v, 1.0, torch.ones(1, dtype=F), torch.full((1,), -1e9, dtype=F))
    assert torch.allclose(out[:, 0, 0], torch.tensor([2.0, 3.0, 6.0], dtype=F))
    x = torch.tensor([[1.0], [2.0], [3.0]], dtype=F)
    y = plain.causal_conv_silu(x, torch.tensor([[10.0, 1.0]], dtype=F))          # the last column weighs the current token
    z = torch.tensor([1.0, 12.0, 23.0], dtype=F)
    assert torch.allclose(y[:, 0], z * torch.sigmoid(z))
    r = plain.rotate_half_pairs(torch.tensor([[[1.0, 5.0, 0.0, 7.0]]], dtype=F), torch.tensor([1]), 2, 10.0)
    # the first two elements turn together by the angle 1 (dims 2: pairs (0, 1)); the rest passes
    assert torch.allclose(r[0, 0], torch.tensor([torch.cos(torch.tensor(1.0)) - 5 * torch.sin(torch.tensor(1.0)),
                                                 5 * torch.cos(torch.tensor(1.0)) + torch.sin(torch.tensor(1.0)), 0.0, 7.0], dtype=F))


def test_plain_shared_layer_runs_the_owner_s_weights(tmp_path):
    folder = write_model(config([delta(ff=20), shared(delta(ff=20), 0)]), str(tmp_path / "m"))
    cfg, w = plain.read_model(folder)
    trace = []
    plain.forward(cfg, w, [3, 9, 27, 1], trace)
    cfg1 = json.loads(json.dumps(cfg))
    cfg1["layers"] = cfg1["layers"][:1]
    first = []
    plain.forward(cfg1, w, [3, 9, 27, 1], first)
    assert torch.equal(trace[0], first[0]) and not torch.allclose(trace[1], trace[0])
