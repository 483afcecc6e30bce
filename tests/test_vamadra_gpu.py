"""The Vamadra design in the engine against the plain implementation of tests/plain_vamadra.py.

Every test makes its own small configuration and random weights (tests/vamadra_cases.py), writes a model folder with
the engine's random-weights mode, reads it back with the plain reader, and compares logits: float32 to 2e-4 of the
largest logit, bfloat16 to 6e-2 (tiny widths average little out).  In float32 the rows of every cut must also EQUAL
the rows of the whole request bit for bit: the 32-bit kernels take a token's sums in an order that depends on its
position only.
"""
import os

import numpy as np
import pytest
import torch

import plain_vamadra as plain
from vamadra_cases import CASES, SINGLE, Harness, config, dense, layer, moe, rel_err, rot, write_model

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def plain_logits(folder, tokens):
    cfg, w = plain.read_model(folder)
    return plain.forward(cfg, w, list(tokens)).numpy()


def plain_rows(folder, tokens, dtype="bfloat16"):
    """The plain logits and which rows to compare.  A token whose router's call is close (the gap between what is chosen
    and what is not below 2 % of the size of a logit's terms) may go to another expert once the activations are rounded to bfloat16,
    and its row then differs as a whole; such rows are left out in bfloat16.  float32 keeps every row."""
    cfg, w = plain.read_model(folder)
    margins = []
    want = plain.forward(cfg, w, list(tokens), margins=margins).numpy()
    clear = np.ones(len(tokens), dtype=bool)
    if dtype != "float32":
        for per_token in margins:
            clear &= np.array(per_token) >= 0.02
    return want, clear


def err(got, want, clear=None):
    d = np.abs(got - want)
    return float((d if clear is None else d[clear]).max() / np.abs(want).max())


def tokens_of(rng, n, vocab):
    return rng.integers(0, vocab, n).tolist()


# ---- each mechanism alone: kernels ----------------------------------------------------------------
def test_norm_of_a_sublayers_output_added_into_the_residual():
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(1)
    for T, W in ((5, 48), (1, 36), (70, 257), (9, 512), (3, 260)):
        y, x, w = torch.randn(T, W, generator=g) * 4, torch.randn(T, W, generator=g), torch.randn(W, generator=g) * 0.1
        want = x.double() + plain.norm_zero_centred(y.double(), w.double(), 1e-5)
        xd = x.cuda()
        ops.rmsnorm_add(y.cuda(), (1.0 + w).cuda(), xd, 1e-5)
        assert rel_err(xd.cpu().numpy(), want.numpy()) < 1e-6
        # with the rounded copy that the next sublayer reads: the same residual, and its rounding
        xd2, rounded = x.cuda(), torch.zeros(T, W, dtype=torch.bfloat16, device="cuda")
        ops.rmsnorm_add(y.cuda(), (1.0 + w).cuda(), xd2, 1e-5, rounded)
        assert torch.equal(xd2, xd) and torch.equal(rounded, xd.bfloat16())


def test_router_kernel_picks_what_the_plain_router_picks():
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(2)
    for T, E, top, groups, keep, scale, gate in ((9, 6, 2, 3, 2, 1.7, True), (4, 8, 4, 2, 1, 2.5, True), (33, 5, 3, 5, 4, 1.0, False),
                                                 (7, 7, 7, 1, 1, 1.0, False), (3, 64, 6, 8, 3, 0.5, True), (5, 4, 1, 1, 1, 1.0, False),
                                                 (6, 12, 3, 12, 3, 3.0, True), (2, 300, 8, 1, 1, 1.0, False)):
        z = torch.randn(T, E + (1 if gate else 0) + 3, generator=g) * 2          # a wider row than the router needs
        ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(T, top, device="cuda")
        sg = torch.empty(T, device="cuda") if gate else None
        ops.moe_route(z.cuda(), E, top, groups, keep, scale, ids, wts, sg)
        router = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}
        for t in range(T):
            chosen, weights = plain.route(z[t, :E].double(), router)
            assert ids[t].tolist() == chosen, (E, top, groups, keep, t)
            assert np.allclose(wts[t].cpu().numpy(), weights, rtol=2e-5)
        if gate:
            assert torch.allclose(sg.cpu(), torch.sigmoid(z[:, E]), atol=1e-6)
    # a group wins by its LARGEST member, not by its sum: group 0 has the single best expert, group 1 the larger sum
    z = torch.tensor([[4.0, -9.0, -9.0, 3.0, 3.0, 3.0]])
    ids, wts = torch.empty(1, 2, dtype=torch.int32, device="cuda"), torch.empty(1, 2, device="cuda")
    ops.moe_route(z.cuda(), 6, 2, 2, 1, 1.0, ids, wts)
    assert ids[0].tolist() == [0, 1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_products_over_the_layout_by_expert(dtype):
    """Route, lay out by expert, the two grouped products, the weighted sum and the gated shared expert, as kernels one
    after another, against the plain loop over tokens and experts; with tiles of 16 and of 64 rows, experts that get no
    token, and (bfloat16, sizes in multiples of 16) the tensor-core product."""
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(3)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for T, W, E, top, ff, sff, tile in ((13, 40, 6, 2, 12, 20, 16), (70, 48, 4, 3, 32, 16, 64), (3, 32, 16, 2, 16, 48, 16),
                                        (150, 64, 5, 1, 24, 0, 64), (1, 36, 8, 8, 7, 5, 16)):
        rnd = lambda *s: (torch.randn(*s, generator=g) * 0.4).to(dtype).double()
        h = rnd(T, W)
        w = {"m.router": rnd(E, W) * 3}
        for e in range(E):
            w[f"m.e{e}.up"], w[f"m.e{e}.down"] = rnd(ff, W), rnd(W, ff)
        mlp = {"router": {"experts": E, "top": top, "scale": 1.3}}
        if sff:
            w["m.shared.up"], w["m.shared.down"], w["m.shared.sg"] = rnd(sff, W), rnd(W, sff), rnd(1, W)
            mlp["shared"] = {"ff": sff}
        want = plain.moe_ffn(w, "m", mlp, h)
        dev = lambda t: t.to(dtype).cuda().contiguous()
        z = torch.zeros(T, E + 1, device="cuda")
        z[:, :E] = (h @ w["m.router"].T).float().cuda()
        if sff:
            z[:, E] = (h @ w["m.shared.sg"].T).float().cuda()[:, 0]
        ids, wts = torch.empty(T, top, dtype=torch.int32, device="cuda"), torch.empty(T, top, device="cuda")
        sg = torch.empty(T, device="cuda") if sff else None
        ops.moe_route(z, E, top, 1, 1, 1.3, ids, wts, sg)
        tiles = ops.moe_max_tiles(T * top, E, tile)
        i32 = lambda n: torch.full((n,), -7, dtype=torch.int32, device="cuda")
        row_token, pair_row, tile_expert, n_tiles = i32(tiles * tile), i32(T * top), i32(tiles), i32(1)
        ops.moe_align(ids, E, tile, row_token, pair_row, tile_expert, n_tiles)
        n = int(n_tiles[0])
        rt, pr, te = row_token.cpu().numpy(), pair_row.cpu().numpy(), tile_expert.cpu().numpy()
        flat = ids.cpu().numpy().reshape(-1)
        assert 0 < n <= tiles and sorted(pr.tolist()) == sorted(set(pr.tolist()))          # every pair a row of its own
        for i, p in enumerate(pr):
            assert rt[p] == i // top and te[p // tile] == flat[i] and p < n * tile
        assert (rt[:n * tile] >= 0).sum() == T * top and set(rt[:n * tile][rt[:n * tile] < 0].tolist()) <= {-1}
        up = dev(torch.stack([w[f"m.e{e}.up"] for e in range(E)]))
        down = dev(torch.stack([w[f"m.e{e}.down"] for e in range(E)]))
        hd = dev(h)
        act = torch.empty(tiles * tile, ff, dtype=dtype, device="cuda")
        ops.reset_kernel_counts()
        ops.moe_matmul(hd, up, act, tile, "relu2", row_token, tile_expert, n_tiles)
        rows = torch.empty(tiles * tile, W, dtype=dtype, device="cuda")
        ops.moe_matmul(act, down, rows, tile, "none", None, tile_expert, n_tiles)
        tensor_cores = dtype == torch.bfloat16 and W % 16 == 0 and ff % 16 == 0
        assert ("moe_matmul_wmma_kernel" in ops.kernel_counts()) == tensor_cores
        shared = None
        if sff:
            sact = torch.empty(T, sff, dtype=dtype, device="cuda")
            ops.moe_matmul(hd, dev(w["m.shared.up"]).unsqueeze(0), sact, tile, "relu2")
            shared = torch.empty(T, W, dtype=dtype, device="cuda")
            ops.moe_matmul(sact, dev(w["m.shared.down"]).unsqueeze(0), shared, tile, "none")
        y = torch.full((T, W), 0.5, device="cuda")
        ops.moe_combine(rows, pair_row, wts, y, shared, sg, True)
        assert rel_err(y.cpu().numpy() - 0.5, want.numpy()) < tol, (T, W, E, top)
        ops.moe_combine(rows, pair_row, wts, y, shared, sg, False)
        assert rel_err(y.cpu().numpy(), want.numpy()) < tol


def test_experts_products_on_the_tensor_core_kernel_that_loads_by_tma():
    """The grouped product in bfloat16 (tiles of 16 and 32 rows as steps of single tokens take them, of 64 and 128 rows for
    steps of many tokens): the tokens' rows copied into the
    layout's order, then both products, against float64; output widths that are no multiple of the kernel's 128 features
    (an expert's last box then reaches into the next expert's rows), depths that are no multiple of 64, experts without a
    token, more tiles allotted than live; and one expert's product over rows as they lie (the shared expert)."""
    from carbon_engine_b200 import ops, ops_tensor
    g = torch.Generator().manual_seed(5)
    for T, W, E, top, ff, tile in ((300, 64, 5, 2, 200, 64), (700, 136, 3, 1, 72, 128), (90, 256, 12, 3, 128, 64), (513, 128, 6, 4, 264, 128),
                                   (4, 64, 9, 2, 96, 16), (21, 200, 7, 3, 40, 32), (1, 128, 5, 4, 136, 16)):
        h = (torch.randn(T, W, generator=g) * 0.5).bfloat16().cuda()
        up = (torch.randn(E, ff, W, generator=g) * 0.3).bfloat16().cuda()
        down = (torch.randn(E, W, ff, generator=g) * 0.3).bfloat16().cuda()
        ids = torch.stack([torch.randperm(E - 1, generator=g)[:top] for _ in range(T)]).int().cuda()      # the last expert gets nothing
        tiles = ops.moe_max_tiles(T * top, E, tile)
        i32 = lambda n: torch.full((n,), -7, dtype=torch.int32, device="cuda")
        row_token, pair_row, tile_expert, n_tiles = i32(tiles * tile), i32(T * top), i32(tiles), i32(1)
        ops.moe_align(ids, E, tile, row_token, pair_row, tile_expert, n_tiles)
        assert int(n_tiles[0]) <= tiles
        laid = torch.full((tiles * tile, W), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.moe_gather(h, row_token, n_tiles, tile, laid)
        live = int(n_tiles[0]) * tile
        rt = row_token[:live].long()
        want_laid = torch.where((rt >= 0)[:, None], h[rt.clamp(min=0)], torch.zeros((), dtype=torch.bfloat16, device="cuda"))
        assert torch.equal(laid[:live], want_laid)
        ops.reset_kernel_counts()
        act = torch.full((tiles * tile, ff), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert ops_tensor.grouped_bf16(laid, up, act, tile, 1, tile_expert, n_tiles)
        rows = torch.full((tiles * tile, W), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert ops_tensor.grouped_bf16(act, down, rows, tile, 0, tile_expert, n_tiles)
        assert ops.kernel_counts().get("gemm_tc_grouped_kernel") == 2
        assert ops_tensor.gemm_status(h.device) == 0
        pr, flat = pair_row.long(), ids.reshape(-1).long()
        a64 = torch.clamp(torch.einsum("pk,pnk->pn", h.double()[torch.arange(T * top, device="cuda") // top], up.double()[flat]), min=0) ** 2
        assert rel_err(act[pr].float().cpu().numpy(), a64.cpu().numpy()) < 1e-2
        r64 = torch.einsum("pk,pnk->pn", act[pr].double(), down.double()[flat])
        assert rel_err(rows[pr].float().cpu().numpy(), r64.cpu().numpy()) < 1e-2
        # one expert over the rows as they lie, a ragged last tile
        one = torch.full((T, ff), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert ops_tensor.grouped_bf16(h, up[1:2].contiguous(), one, tile, 1)
        want = torch.clamp(h.double() @ up[1].double().T, min=0) ** 2
        assert rel_err(one.float().cpu().numpy(), want.cpu().numpy()) < 1e-2
    # sizes the kernel refuses go to the other kernels
    assert not ops_tensor.grouped_bf16_supported(64, 40, 36, 36, 40, torch.bfloat16)
    assert not ops_tensor.grouped_bf16_supported(64, 64, 64, 64, 64, torch.float32)
    assert not ops_tensor.grouped_bf16_supported(48, 64, 64, 64, 64, torch.bfloat16)


def test_squared_relu_as_the_epilogue_of_every_product_kernel():
    """The shared expert's first product: relu(x W^T)^2 from the float32 kernel, the tcgen05 kernels (one block, split
    depth, CTA pairs) and the library product followed by the activation's own kernel."""
    from carbon_engine_b200 import ops, ops_tensor
    from carbon_engine_b200.parts import linear
    g = torch.Generator().manual_seed(6)
    for M, N, K in ((5, 24, 40), (8, 256, 4096), (70, 136, 64), (300, 512, 128), (1000, 384, 256)):
        a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) * 0.2
        want = (torch.relu(a.double() @ w.double().T) ** 2).numpy()
        out = torch.empty(M, N, device="cuda")
        ops.gemm_plain(a.cuda(), w.cuda(), out, ops.GEMM_RELU2)
        assert rel_err(out.cpu().numpy(), want) < 1e-5
        ab, wb = a.cuda().bfloat16(), w.cuda().bfloat16()
        wantb = (torch.relu(ab.double() @ wb.double().T) ** 2).cpu().numpy()
        outb = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        assert ops_tensor.gemm_bf16(ab, wb, outb, ops.GEMM_RELU2)
        assert rel_err(outb.float().cpu().numpy(), wantb) < 1e-2
        outb.zero_()
        linear.BF16_BACKEND = "library"
        try:
            linear.matmul_nt(ab, wb, outb, linear.RELU2)
        finally:
            linear.BF16_BACKEND = "auto"
        assert rel_err(outb.float().cpu().numpy(), wantb) < 1e-2


def test_gate_per_head_on_the_product_per_head():
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(4)
    for T, H, N, K, dtype in ((5, 3, 20, 14, torch.float32), (33, 2, 48, 32, torch.bfloat16), (1, 5, 16, 96, torch.bfloat16)):
        x = torch.randn(T, H * K, generator=g).to(dtype)
        w = (torch.randn(H, N, K, generator=g) * 0.3).to(dtype)
        gate = torch.randn(T, H + 3, generator=g)
        want = torch.einsum("thk,hnk->thn", x.double().reshape(T, H, K), w.double()) * torch.sigmoid(gate[:, :H].double())[:, :, None]
        out = torch.zeros(T, H * N, device="cuda", dtype=dtype)
        ops.head_matmul(x.cuda(), K, w.cuda(), out, N, H, N, K, gate=gate.cuda(), gate_per_head=True)
        assert rel_err(out.float().cpu().numpy(), want.reshape(T, -1).numpy()) < (1e-5 if dtype == torch.float32 else 1e-2)


# ---- each mechanism alone: one layer of each kind ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_layer_of_each_kind(tmp_path, name, dtype):
    folder = write_model(SINGLE[name], str(tmp_path / name), seed=7)
    rng = np.random.default_rng(5)
    toks = tokens_of(rng, 45, SINGLE[name]["vocab"])
    want, clear = plain_rows(folder, toks, dtype)
    assert clear.sum() > 30
    h = Harness(folder, dtype)
    whole = h.run(toks)
    assert err(whole, want, clear) < TOL[dtype]
    one_by_one = h.run(toks, [1])
    assert err(one_by_one, want, clear) < TOL[dtype]
    if dtype == "float32":
        assert np.array_equal(whole, one_by_one)


def test_layers_outputs_one_after_another(tmp_path):
    """The residual after every layer, in float32."""
    from carbon_engine_b200.engine.batch import StepEntry
    for name in ("A", "B"):
        folder = write_model(CASES[name], str(tmp_path / name))
        cfg, w = plain.read_model(folder)
        toks = tokens_of(np.random.default_rng(1), 30, cfg["vocab"])
        trace = []
        plain.forward(cfg, w, toks, tap=lambda i, x: trace.append(x.clone()))
        h = Harness(folder, "float32")
        rid = h.open()
        ctx, rows, commits = h.runner.prepare([StepEntry(rid, toks, [0])])
        got = []
        h.model.forward(ctx, h.storage, tap=lambda i, x: got.append(x.clone().cpu().numpy()))
        assert len(got) == len(trace) == 4
        for i, (a, b) in enumerate(zip(got, trace)):
            assert rel_err(a.reshape(b.shape), b.numpy()) < 1e-4, (name, i)


def test_the_sink_and_the_gate_show_in_the_logits(tmp_path):
    """Sinks of either sign and size: the plain model without them gives other logits (so a sink left out would show),
    and the engine follows the plain model with them; the same for the gate per head."""
    from helpers import read_raw_safetensors, write_safetensors_plain
    raw = config([layer(heads=3, mlp=None), layer(heads=3, kv_from=0, mlp=None)])
    folder = write_model(raw, str(tmp_path / "sinks"), seed=31)
    path = os.path.join(folder, "model.safetensors")
    t = read_raw_safetensors(path)
    t["l0.mix.sink"] = torch.tensor([3.0, -2.0, 0.5]).to(t["l0.mix.sink"].dtype)
    t["l1.mix.sink"] = torch.tensor([-30.0, 6.0, 1.0]).to(t["l1.mix.sink"].dtype)
    t["l0.mix.g"] = t["l0.mix.g"] * 6.0
    write_safetensors_plain(path, t)
    cfg, w = plain.read_model(folder)
    toks = tokens_of(np.random.default_rng(2), 70, raw["vocab"])
    want = plain.forward(cfg, w, toks).numpy()
    # (a gate that is equal for all heads would be undone by the norm on the mixer's output: the heads' gates are swapped)
    for name, other_value in (("l0.mix.sink", torch.full((3,), -1e9, dtype=torch.float64)),
                              ("l1.mix.sink", torch.full((3,), -1e9, dtype=torch.float64)), ("l0.mix.g", -w["l0.mix.g"])):
        other = dict(w)
        other[name] = other_value
        moved = np.abs(plain.forward(cfg, other, toks).numpy() - want).max(axis=1) / np.abs(want).max()
        # the sinks at every position, the first one too; the gates at most (a token's gates may all be near one half)
        assert (np.median(moved) if name.endswith(".g") else moved.min()) > 5e-3, name
    for dtype in ("float32", "bfloat16"):
        h = Harness(folder, dtype)
        assert rel_err(h.run(toks), want) < TOL[dtype]
        assert rel_err(h.run(toks, [1]), want) < TOL[dtype]
        assert rel_err(h.run(toks, [5, 2, 64]), want) < TOL[dtype]


# ---- whole models: cuts, batches, reuse ------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_whole_prompt_portions_and_decoding(tmp_path, name, dtype):
    from carbon_engine_b200 import ops
    folder = write_model(CASES[name], str(tmp_path / name), seed=11)
    rng = np.random.default_rng(3)
    toks = tokens_of(rng, 83, CASES[name]["vocab"])
    want, clear = plain_rows(folder, toks, dtype)
    assert clear.sum() > 60
    h = Harness(folder, dtype, page_size=8, pages=16)          # 128 tokens of pages: every run reuses the last one's
    ops.reset_kernel_counts()
    whole = h.run(toks)
    if name in ("T", "V"):           # sizes of the tensor-core kernels: bfloat16 must have taken them, float32 never
        counts = ops.kernel_counts()
        assert ("masked_attention_mma_kernel" in counts) == (dtype == "bfloat16")
        assert ("gemm_tc_grouped_kernel" in counts) == (dtype == "bfloat16")
    assert err(whole, want, clear) < TOL[dtype], "whole"
    for cuts in ([1], [2], [3, 2, 7, 2, 16, 5], [40, 1, 1, 1], [64, 19]):
        got = h.run(toks, cuts)
        assert err(got, want, clear) < TOL[dtype], cuts
        if dtype == "float32":
            assert np.array_equal(got, whole), cuts
    if name in ("T", "V"):           # single tokens take the same kernel with small tiles; float32 never
        assert ("moe_matmul_plain_kernel" in ops.kernel_counts()) == (dtype == "float32")
    assert h.storage.manager.free_slots() == 4
    assert all(h.storage.manager.free_pages(g) == 16 for g in range(len(h.storage.groups)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "T"])
def test_unequal_requests_in_one_batch_with_reused_pages_and_slots(tmp_path, name, dtype):
    """Up to three live requests, portions beside single tokens, a request left out of some steps, finished requests'
    pages and slots taken by the next: every row equals the request alone."""
    folder = write_model(CASES[name], str(tmp_path / name), seed=13)
    rng = np.random.default_rng(9)
    lengths = [61, 17, 40, 1, 2, 33, 25]
    reqs = [tokens_of(rng, n, CASES[name]["vocab"]) for n in lengths]
    want = [plain_rows(folder, t, dtype) for t in reqs]
    h = Harness(folder, dtype, page_size=8, pages=20, slots=3)          # 160 tokens: three live requests at most
    alone = [h.run(t) for t in reqs] if dtype == "float32" else None
    waiting, live, done_rows = list(range(len(reqs))), {}, {i: [] for i in range(len(reqs))}
    portions, k, step_no = [2, 5, 1, 9, 3, 14], 0, 0
    while waiting or live:
        while waiting and len(live) < 3 and sum(-(-len(reqs[i]) // 8) for i in live) + -(-len(reqs[waiting[0]]) // 8) <= 20:
            i = waiting.pop(0)
            live[i] = [h.open(), 0]
        entries, who = [], []
        for i, (rid, pos) in list(live.items()):
            if step_no % 4 == 3 and i % 2 == 0 and len(live) > 1:
                continue                                     # left out of this step
            left = len(reqs[i]) - pos
            n = 1 if left <= 6 else min(portions[k % len(portions)], left - 6)      # the last tokens one by one
            k += 1
            entries.append((rid, reqs[i][pos:pos + n], range(n)))
            who.append((i, n))
        step_no += 1
        if not entries:
            continue
        rows = h.step(entries)
        at = 0
        for i, n in who:
            done_rows[i].append(rows[at:at + n])
            at += n
            live[i][1] += n
            if live[i][1] == len(reqs[i]):
                h.close(live.pop(i)[0])
    for i in range(len(reqs)):
        got = np.concatenate(done_rows[i])
        assert err(got, *want[i]) < TOL[dtype], i
        if alone is not None:
            assert np.array_equal(got, alone[i]), i
    assert h.storage.manager.free_slots() == 3
    assert all(h.storage.manager.free_pages(g) == 20 for g in range(len(h.storage.groups)))


# ---- keys that stand out: far away, at page borders, among the first tokens ----------------------------------------
def standout_model(tmp_path, tag, reader=False, heads=2):
    """One latent-attention layer (or a writer and a reader of its rows) in which EVERY query scores the marker token's
    key far above hundreds of others.  The sublayers read the residual itself, so in layer 0 a token's input is its
    embedding: element 0 of every embedding is made 1, one unrotated element of every query head reads it (a constant),
    the first element of the latent reads the direction of the marker's embedding (large for the marker, noise for all
    others), and the same unrotated element of every key head reads that first latent element."""
    from helpers import read_raw_safetensors, write_safetensors_plain
    W, d, dr, r, j = 32, 16, 4, 24, 10
    mixer = dict(heads=heads, dim=d, rot_dim=dr, vdim=16, kv_rank=r, scale=0.6, rotation=rot(dims=4, base=100.0, factor=2.0, original=64, fast=4.0))
    layers = [layer(mlp=None, **mixer)] + ([layer(mlp=None, kv_from=0, **mixer)] if reader else [])
    raw = config(layers, width=W, vocab=50)
    folder = write_model(raw, str(tmp_path / f"standout_{tag}"), seed=21)
    path = os.path.join(folder, "model.safetensors")
    t = read_raw_safetensors(path)
    t["embed"][:, 0] = 1.0
    e = t["embed"][7].float().clone()
    e[0] = 0.0
    t["embed"][7] = (t["embed"][7].float() * 3.0).to(t["embed"].dtype)
    t["embed"][7, 0] = 1.0
    t["l0.mix.dkv"][0] = (2.0 * e / e.norm()).to(t["l0.mix.dkv"].dtype)
    t["l0.mix.dkv.norm"] = torch.ones(r).to(t["l0.mix.dkv.norm"].dtype)
    for i in range(len(layers)):
        # in the reader the residual has moved on, but its element 0 still holds about 1
        for head in range(heads):
            t[f"l{i}.mix.q"][head * (d + dr) + j] = 0.0
            t[f"l{i}.mix.q"][head * (d + dr) + j, 0] = 2.0
            t[f"l{i}.mix.uk"][head * d + j] = 0.0
            t[f"l{i}.mix.uk"][head * d + j, 0] = 2.0
        t[f"l{i}.mix.sink"] = torch.zeros(heads).to(t[f"l{i}.mix.sink"].dtype)
    write_safetensors_plain(path, t)
    return folder, raw


def marker_effect(folder, toks, at):
    """How far the plain model's rows move when the marker at ``at`` is replaced by an ordinary token."""
    want = plain_logits(folder, toks)
    other = list(toks)
    other[at] = 9
    return want, np.abs(want - plain_logits(folder, other)).max(axis=1) / np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("reader", [False, True])
def test_a_key_that_stands_out_at_page_and_tile_borders(tmp_path, reader, dtype):
    """The marker as the first token, as the last and first row of a page, of a tile of 64 keys, and in between: every
    later query sees it (and none before it), met in a portion's middle, at its start, and by single tokens."""
    folder, raw = standout_model(tmp_path, f"near{int(reader)}", reader)
    rng = np.random.default_rng(4)
    base = [int(t) for t in rng.integers(10, 50, 150)]
    h = Harness(folder, dtype, page_size=8, pages=64)
    for marker_at in (0, 1, 7, 8, 63, 64, 100):
        toks = list(base)
        toks[marker_at] = 7
        want, moved = marker_effect(folder, toks, marker_at)
        assert moved[marker_at:].min() > 1e-3 and (marker_at == 0 or moved[:marker_at].max() < 1e-9)
        whole = h.run(toks)
        assert rel_err(whole, want) < TOL[dtype], marker_at
        for cuts in ([max(marker_at, 1), 1, 1, 1, 1, 40], [marker_at + 1, 2, 2, 50], [marker_at + 2, 64], [13], [1]):
            got = h.run(toks, cuts)
            assert rel_err(got, want) < TOL[dtype], (marker_at, cuts)
            if dtype == "float32":
                assert np.array_equal(got, whole)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("reader", [False, True])
def test_a_far_key_among_hundreds(tmp_path, reader, dtype):
    """The marker near the start must still carry its weight 700 tokens later, in a prompt and in decoding, across many
    pages; also for the layer that reads another layer's rows."""
    folder, raw = standout_model(tmp_path, f"far{int(reader)}", reader, heads=4)
    rng = np.random.default_rng(6)
    toks = [int(t) for t in rng.integers(10, 50, 720)]
    toks[3] = 7
    want, moved = marker_effect(folder, toks, 3)
    assert moved[700:].min() > 1e-2                       # the plain model says the far key matters
    h = Harness(folder, dtype, page_size=16, pages=48, max_step_tokens=1024)
    assert rel_err(h.run(toks), want) < TOL[dtype]
    rid = h.open()
    rows = [h.step([(rid, toks[:690], [689])])]
    for p in range(690, 720):
        rows.append(h.step([(rid, toks[p:p + 1], [0])]))
    h.close(rid)
    assert rel_err(np.concatenate(rows), want[689:]) < TOL[dtype]


def test_long_decoding_keeps_the_cache(tmp_path):
    """300 tokens one by one after a short prompt, in float32: the writers' rows must carry every token for themselves and
    for their readers (bit for bit the rows of the whole prompt)."""
    folder = write_model(CASES["A"], str(tmp_path / "A"), seed=2)
    toks = tokens_of(np.random.default_rng(8), 310, CASES["A"]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, "float32", page_size=8, pages=48)
    whole = h.run(toks)
    got = h.run(toks, [10] + [1] * 300)
    assert rel_err(got, want) < TOL["float32"] and np.array_equal(got, whole)
    hb = Harness(folder, "bfloat16", page_size=8, pages=48)
    want, clear = plain_rows(folder, toks)
    assert clear.sum() > 200 and err(hb.run(toks, [10] + [1] * 300), want, clear) < TOL["bfloat16"]


def test_first_tokens_of_a_sequence_in_a_reused_slot(tmp_path):
    """A slot and pages that held a longer request: the next request's first tokens must see no key of it (at position 0
    the softmax holds the token's own key and the sink, nothing else)."""
    folder = write_model(CASES["B"], str(tmp_path / "B"), seed=5)
    rng = np.random.default_rng(12)
    h = Harness(folder, "float32", page_size=8, pages=12, slots=1, poison=False)
    h.run(tokens_of(rng, 90, CASES["B"]["vocab"]))
    for n in (1, 2, 3, 9):
        toks = tokens_of(rng, n, CASES["B"]["vocab"])
        want = plain_logits(folder, toks)
        assert rel_err(h.run(toks), want) < TOL["float32"]
        assert rel_err(h.run(toks, [1]), want) < TOL["float32"]


# ---- through the entry point -------------------------------------------------------------------------
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(tmp_path, graphs):
    from carbon_engine_b200 import Engine, SamplingParams
    folder = write_model(CASES["A"], str(tmp_path / "A"), seed=17)
    cfg, w = plain.read_model(folder)
    rng = np.random.default_rng(2)
    prompts = [tokens_of(rng, n, cfg["vocab"]) for n in (23, 5, 41)]
    eng = Engine(folder, dtype="float32", page_size=8, max_running_requests=3, max_prefill_tokens=16, kv_tokens=256,
                 cuda_graphs=graphs)
    assert eng.cuda_graphs == graphs
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out.token_ids) == 12 and out.finish_reason == "length"
        toks = list(prompt)
        for t in out.token_ids:
            row = plain.forward(cfg, w, toks)[-1]
            assert t == int(row.argmax()) or float(row.max() - row[t]) < 4e-4 * float(row.abs().max())
            toks.append(t)
    eng.storage.manager.check()


def test_greedy_generation_in_bfloat16_with_graphs(tmp_path):
    """The serving configuration (bfloat16, captured decode steps, the tensor-core kernels) on sizes they take: every
    generated token is the plain model's best or within bfloat16's reach of it."""
    from carbon_engine_b200 import Engine, SamplingParams
    folder = write_model(CASES["T"], str(tmp_path / "T"), seed=19)
    cfg, w = plain.read_model(folder)
    rng = np.random.default_rng(3)
    prompts = [tokens_of(rng, n, cfg["vocab"]) for n in (70, 9, 33, 2)]
    eng = Engine(folder, dtype="bfloat16", page_size=16, max_running_requests=4, max_prefill_tokens=64, kv_tokens=512, cuda_graphs=True)
    outs = eng.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        toks = list(prompt)
        for t in out.token_ids:
            margins = []
            row = plain.forward(cfg, w, toks, margins=margins)[-1]
            if all(per_token[-1] >= 0.02 for per_token in margins):        # (a close router call may go either way)
                assert float(row.max() - row[t]) < 6e-2 * float(row.abs().max())
            toks.append(t)
    eng.storage.manager.check()


def test_trace_replay_program_on_a_vamadra_folder(tmp_path):
    import json, subprocess, sys
    from helpers import ROOT
    folder = write_model(CASES["B"], str(tmp_path / "B"), seed=1)
    toks = tokens_of(np.random.default_rng(3), 40, CASES["B"]["vocab"])
    want = plain_logits(folder, toks)
    out = str(tmp_path / "out")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[25:27], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[27:], "want": [12]}, {"id": "b", "tokens": toks[:3], "want": [2]}],
              "end": ["a", "b"]}]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                           "--out", out, "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    got0 = np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(2, -1)
    got2 = np.fromfile(os.path.join(out, "2.f32"), dtype="<f4").reshape(2, -1)
    assert not os.path.exists(os.path.join(out, "1.f32"))
    assert rel_err(got0, want[[0, 24]]) < 2e-4 and rel_err(got2, want[[39, 2]]) < 2e-4


def test_command_line_writes_and_generates_a_vamadra_model(tmp_path):
    """``tiny-model --arch vamadra`` then ``generate``: the printed ids are the plain implementation's greedy ones."""
    import ast, re, subprocess, sys
    from helpers import ROOT
    carbon = [sys.executable, os.path.join(ROOT, "bin", "carbon")]
    out = str(tmp_path / "tiny_v")
    p = subprocess.run(carbon + ["tiny-model", "--arch", "vamadra", "--out", out, "--layers", "4", "--hidden", "48", "--heads", "3",
                                 "--head-dim", "12", "--vocab", "120", "--seed", "9", "--experts", "6", "--top-experts", "2",
                                 "--expert-groups", "3", "--yarn-factor", "2.0", "--max-positions", "256"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "wrote" in p.stdout, p.stderr[-2000:]
    cfg, w = plain.read_model(out)
    assert cfg["architecture"] == "Vamadra" and len(cfg["layers"]) == 4 and cfg["layers"][1]["mixer"]["kv_from"] == 0
    assert cfg["layers"][1]["mlp"]["kind"] == "moe" and cfg["layers"][0]["mixer"]["rot"]["scaling"]["factor"] == 2.0
    prompt = tokens_of(np.random.default_rng(5), 17, 120)
    p = subprocess.run(carbon + ["generate", "--model", out, "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "8",
                                 "--ignore-eos", "--print-ids", "--dtype", "f32", "--kv-tokens", "256", "--page-size", "16"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ids = [ast.literal_eval(m) for m in re.findall(r"output_ids: (\[[^\]]*\])", p.stderr)][0]
    toks = list(prompt)
    for t in ids:
        row = plain.forward(cfg, w, toks)[-1]
        assert t == int(row.argmax()) or float(row.max() - row[t]) < 4e-4 * float(row.abs().max())
        toks.append(t)
    assert len(ids) == 8
