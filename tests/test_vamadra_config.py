"""What needs no GPU of the Vamadra design: reading its config.json, which layers write cache rows and which read
another's, the cache its blocks ask for, tensor names, and the plain implementation's own consistency."""
import json
import math
import os

import pytest
import torch

import plain_vamadra as plain
from vamadra_cases import CASES, SINGLE, config, dense, layer, moe, rot, write_model


def test_config_round_trip_and_registry(tmp_path):
    from carbon_engine_b200.config.registry import load_config
    from carbon_engine_b200.config.vamadra import VamadraConfig
    for name, raw in list(CASES.items()) + list(SINGLE.items()):
        folder = write_model(raw, str(tmp_path / name))
        arch, cfg = load_config(folder)
        assert arch.name == "Vamadra" and cfg == VamadraConfig.from_dict(json.loads(json.dumps(raw)))
        with open(os.path.join(folder, "config.json")) as fh:
            assert VamadraConfig.from_dict(json.load(fh)) == cfg
        # the plain reader takes the folder the engine wrote
        pcfg, w = plain.read_model(folder)
        assert pcfg["vocab"] == raw["vocab"] and w["embed"].shape == (raw["vocab"], raw["width"])


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=64), "at most rot_dim"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "no down-projection"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=10), "must equal"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "dense"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top=9"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=0), "keep"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_config_errors_name_the_key(change, message):
    from carbon_engine_b200.config.base import ConfigError
    from carbon_engine_b200.config.vamadra import VamadraConfig
    raw = json.loads(json.dumps(CASES["A"]))
    change(raw)
    with pytest.raises(ConfigError, match=message):
        VamadraConfig.from_dict(raw)


def test_schedule_caches_and_tensor_names():
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.registry import resolve_architecture
    from carbon_engine_b200.config.vamadra import VamadraConfig
    from carbon_engine_b200.parts.base import PagedCacheSpec
    raw = CASES["B"]
    model = resolve_architecture(raw).build_model(VamadraConfig.from_dict(raw), 256)
    # layer 2 reads what layer 0 cached; 0, 1 and 3 write rows of their own
    assert [(c.block, c.cache, c.writes) for c in model.schedule] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]
    layout = dict(model.cache_layout())
    assert set(layout) == {0, 1, 3}
    # one row of kv_rank + rot_dim per token, no value pool
    assert layout[0] == PagedCacheSpec(1, 9 + 6, 0, None, v_heads=1, v_head_dim=0)
    assert layout[1] == PagedCacheSpec(1, 30 + 2, 0, None, v_heads=1, v_head_dim=0)
    names = {s.name for s in model.all_tensor_specs()}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk",
            "l0.mix.uv", "l0.mix.sink", "l0.mix.g", "l0.mix.o", "l0.mlp.router", "l0.mlp.e4.up", "l0.mlp.e0.down",
            "l0.mlp.shared.up", "l0.mlp.shared.down", "l0.mlp.shared.sg", "l3.mlp.gate", "l3.mlp.up", "l3.mlp.down"} <= names
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names          # a reader has no down-projection
    assert "l1.norm2" not in names and not any(n.startswith("l1.mlp") for n in names)   # no feed-forward, no second norm
    assert "l0.mlp.e5.up" not in names
    shapes = {s.name: tuple(s.shape) for s in model.all_tensor_specs()}
    assert shapes["l2.mix.q"] == (5 * (4 + 6), 36) and shapes["l2.mix.uk"] == (5 * 4, 9) and shapes["l2.mix.uv"] == (5 * 9, 9)
    assert shapes["l2.mix.g"] == (5, 36) and shapes["l2.mix.sink"] == (5,) and shapes["l0.mlp.shared.sg"] == (1, 36)
    assert model.graph_safe
    # a mixture without a shared expert has none of its tensors
    a = resolve_architecture(CASES["A"]).build_model(VamadraConfig.from_dict(CASES["A"]), 64)
    assert not any(s.name.startswith("l3.mlp.shared") for s in a.all_tensor_specs())


def test_cache_storage_holds_rows_for_the_writers_only():
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.cache.storage import CacheStorage
    from carbon_engine_b200.config.registry import resolve_architecture
    from carbon_engine_b200.config.vamadra import VamadraConfig
    raw = CASES["A"]
    model = resolve_architecture(raw).build_model(VamadraConfig.from_dict(raw), 128)
    st = CacheStorage(model, torch.float32, torch.device("cpu"), 8, 10, 3, 128)
    views = [st.view(c) for c in model.schedule]
    assert views[1].k_pool.shape == (10, 1, 8, 14 + 8)
    assert views[2].k_pool.data_ptr() == views[1].k_pool.data_ptr() == views[3].k_pool.data_ptr()
    assert views[0].k_pool.data_ptr() != views[1].k_pool.data_ptr()
    assert views[1].writes and not views[2].writes and not views[3].writes
    assert st.bytes_per_token() == 2 * (14 + 8) * 4                 # two writers, float32


def test_rotary_table_is_the_plain_frequencies():
    """The engine's stretched frequencies and the factor on cos and sin against the plain implementation's, for ramps
    that start at the first pair, end before the last, have no width at all, and for a factor below 1."""
    from carbon_engine_b200.models.vamadra import _rotation
    for r in (rot(dims=8, base=300.0, factor=3.0, original=24, fast=6.0, slow=0.5), rot(dims=16, base=1e4, factor=4.0, original=64, fast=16.0),
              rot(dims=2, base=1e4, factor=0.5, original=16), rot(dims=32, base=5e5, factor=8.0, original=4096, fast=32.0, slow=1.0),
              rot(dims=12, base=50.0, factor=2.0, original=8, fast=1.0, slow=1.0), rot(dims=6, base=77.0)):
        m = {"rot_dim": r["dims"] + 4, "rot": r}
        part = _rotation(m, 300)
        part.prepare(torch.device("cpu"))
        freq, mag = plain.rotary_frequencies(r)
        pos = torch.arange(300, dtype=torch.float64)
        ang = pos[:, None] * torch.tensor(freq, dtype=torch.float64)[None, :]
        assert part.rotary_dim == r["dims"] and part.cos.shape == (300, r["dims"] // 2)
        assert torch.allclose(part.cos.double(), ang.cos() * mag, atol=2e-5)
        assert torch.allclose(part.sin.double(), ang.sin() * mag, atol=2e-5)


def test_plain_pieces_agree_with_themselves():
    """The plain attention with keys and values formed per head equals one written with the products moved to the
    query side; the plain softmax with a sink against its definition; the plain router's groups."""
    g = torch.Generator().manual_seed(0)
    W, H, d, dr, dv, r, T = 10, 2, 3, 4, 5, 6, 7
    m = {"heads": H, "dim": d, "rot_dim": dr, "vdim": dv, "kv_rank": r, "scale": 0.4, "rot": rot(dims=4, base=20.0, factor=2.0, original=4, fast=2.0)}
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64) * 0.5
    w = {"x.q": rnd(H * (d + dr), W), "x.dkv": rnd(r + dr, W), "x.dkv.norm": 1 + rnd(r), "x.uk": rnd(H * d, r), "x.uv": rnd(H * dv, r),
         "x.sink": rnd(H), "x.g": rnd(H, W), "x.o": rnd(W, H * dv)}
    h, pos = rnd(T, W), torch.arange(T)
    kept = {}
    out = plain.latent_attention(w, "x", m, h, pos, 1e-5, kept, 0)
    c, k_rot = kept[0]
    q = (h @ w["x.q"].T).view(T, H, d + dr)
    q_rot = plain.rotate(q[..., d:], pos, m["rot"])
    heads = []
    for i in range(H):
        qa = torch.cat([q[:, i, :d] @ w["x.uk"][i * d:(i + 1) * d], q_rot[:, i]], dim=-1)            # [T, r + dr]
        s = qa @ torch.cat([c, k_rot], dim=-1).T * 0.4
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        e = torch.exp(s)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(w["x.sink"][i]))
        heads.append((p @ c) @ w["x.uv"][i * dv:(i + 1) * dv].T * torch.sigmoid(h @ w["x.g"][i])[:, None])
    assert torch.allclose(out, torch.cat(heads, -1) @ w["x.o"].T, atol=1e-12)
    # a reader takes the writer's rows, not its own input
    out2 = plain.latent_attention(w, "x", dict(m, kv_from=0), h * 2.0, pos, 1e-5, kept, 1)
    assert 1 not in kept and not torch.allclose(out2, out)
    # the sink: one more term in the denominator, once, without a value
    p = plain.sink_softmax(torch.zeros(3, 3, dtype=torch.float64), 0.0)
    assert torch.allclose(p[2], torch.full((3,), 0.25, dtype=torch.float64)) and float(p[0, 0]) == 0.5 and float(p[0, 1]) == 0.0
    # groups: the best expert overall sits in a group that loses to none; an expert of a dropped group is never chosen
    z = torch.tensor([0.0, 5.0, 0.1, 0.2, 4.0, 3.9], dtype=torch.float64)
    chosen, weights = plain.route(z, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}, "scale": 2.0})
    assert chosen == [1, 0] and abs(sum(weights) - 2.0) < 1e-12
    chosen, _ = plain.route(z, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}})
    assert chosen == [1, 4]
    chosen, weights = plain.route(z, {"experts": 6, "top": 3})
    assert chosen == [1, 4, 5] and abs(sum(weights) - 1.0) < 1e-12


def test_sketch_config_and_random_weights(tmp_path):
    from carbon_engine_b200.config.vamadra import sketch_config
    from carbon_engine_b200.weights.loader import write_random_model
    cfg = sketch_config(vocab=90, width=48, n_layers=5, heads=3, head_dim=8, ff=64, experts=6, top=2, groups=(3, 2), yarn_factor=2.0)
    kinds = [(l["mixer"].get("kv_from"), None if l["mlp"] is None else l["mlp"]["kind"]) for l in cfg.layers]
    assert kinds == [(None, "dense"), (0, "moe"), (None, "dense"), (2, "moe"), (None, "dense")]
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=4)
    pcfg, w = plain.read_model(folder)
    logits = plain.forward(pcfg, w, [1, 5, 7, 2])
    assert logits.shape == (4, 90) and bool(torch.isfinite(logits).all())
    # the zero-centred norms' weights are stored around 0, the down-projection's plain norm around 1
    assert abs(float(w["l0.norm1"].mean())) < 0.2 and abs(float(w["l0.mix.dkv.norm"].mean()) - 1.0) < 0.2
