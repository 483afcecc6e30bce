"""The Pugozen design in the engine against the plain implementation of tests/plain_pugozen.py.

Every test makes its own small configuration and random weights (tests/pugozen_cases.py), writes a model folder with
the engine's random-weights mode, reads it back with the plain reader, and compares logits: float32 to 2e-4 of the
largest logit, bfloat16 to 6e-2 (tiny widths average little out).  In float32 the rows of every cut must also EQUAL
the rows of the whole request bit for bit: the 32-bit kernels take a token's sums in an order that depends on its
position only.  The design has no window and no chunk: what a query sees ends at itself, so the edges that matter are
those of pages, of portions, of the convolution's first tokens and of a slot's reuse.
"""
import os

import numpy as np
import pytest
import torch

import plain_pugozen as plain
from pugozen_cases import CASES, SINGLE, Harness, config, delta, pair, rel_err, retention, shared, write_model

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def plain_logits(folder, tokens, layers_out=None):
    cfg, w = plain.read_model(folder)
    return plain.forward(cfg, w, list(tokens), layers_out).numpy()


def tokens_of(rng, n, vocab):
    return rng.integers(0, vocab, n).tolist()


def _step_arrays(lengths, slots):
    """Device arrays of a step whose sequences bring ``lengths`` tokens each."""
    seq = torch.tensor([b for b, n in enumerate(lengths) for _ in range(n)], dtype=torch.int32, device="cuda")
    starts = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32, device="cuda")
    return seq, torch.tensor(slots, dtype=torch.int32, device="cuda"), starts


# ---- each mechanism alone: the kernels --------------------------------------------------------------------
@pytest.mark.parametrize("H, G, d, dv, K", [(3, 3, 12, 8, 1), (4, 2, 8, 12, 4), (2, 1, 136, 8, 2), (2, 2, 10, 7, 3)])
def test_delta_rule_kernels_with_a_decay_per_head(H, G, d, dv, K):
    """Two sequences in two steps (the second continues from the state and the kept convolution inputs) against the walk."""
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + d)
    lengths, C = [7, 3], 2 * G * d + H * dv
    T = sum(lengths)
    off_b = C
    ld = (C + 2 * H + H * dv + 3) // 4 * 4
    taps = torch.randn(C, K, generator=g) * 0.5
    a_log, dt_bias, norm_w = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g) * 0.3, 1 + 0.1 * torch.randn(dv, generator=g)
    state = torch.zeros(3, H, d, dv, device="cuda")
    kept = torch.zeros(3, max(K - 1, 1), C, device="cuda")
    slots = [2, 0]
    seq, slot_t, starts = _step_arrays(lengths, slots)
    rows = [torch.randn(2 * n, ld, generator=g) for n in lengths]            # each sequence's inputs of both steps
    outs = []
    for step in range(2):
        proj = torch.cat([r[step * n:(step + 1) * n] for r, n in zip(rows, lengths)]).cuda()
        prep = torch.empty(T, ops.gated_delta_prep_width(H, G, d, dv), device="cuda")
        raw, out = torch.empty(T, H * dv, device="cuda"), torch.empty(T, H * dv, device="cuda")
        ops.gated_delta(proj, proj[:, off_b + H:off_b + 2 * H], proj[:, off_b + 2 * H:off_b + 2 * H + H * dv], taps.cuda(), a_log.cuda(),
                        dt_bias.cuda(), norm_w.cuda(), prep, raw, state, kept if K > 1 else None, out, seq, slot_t, starts, 2, 0, off_b,
                        H, G, d, dv, K, 1e-5, decay=ops.DECAY_PER_HEAD, gate=ops.GATE_SILU, out_scale=0.75)
        outs.append(out.cpu())
    for b, n in enumerate(lengths):
        x = rows[b].double()
        conv = plain.causal_conv_silu(x[:, :C], taps.double())
        q = plain.unit(conv[:, :G * d].reshape(-1, G, d)) * d ** -0.5
        k = plain.unit(conv[:, G * d:2 * G * d].reshape(-1, G, d))
        v = conv[:, 2 * G * d:].reshape(-1, H, dv)
        beta = torch.sigmoid(x[:, off_b:off_b + H])
        dec = torch.exp(-torch.exp(a_log.double()) * plain.softplus(x[:, off_b + H:off_b + 2 * H] + dt_bias.double()))
        gz = x[:, off_b + 2 * H:off_b + 2 * H + H * dv]
        want = torch.stack([plain.delta_rule_walk(q[:, i // (H // G)], k[:, i // (H // G)], v[:, i], dec[:, i:i + 1].expand(-1, d), beta[:, i])
                            for i in range(H)], dim=1)
        want = (plain.rms_norm(want, norm_w.double(), 1e-5).reshape(2 * n, -1) * plain.silu(gz) * 0.75).numpy()
        at = sum(lengths[:b])
        got = np.concatenate([outs[0][at:at + n].numpy(), outs[1][at:at + n].numpy()])
        assert rel_err(got, want) < 2e-5, b


@pytest.mark.parametrize("delta_rule", [True, False])
def test_the_walk_with_two_columns_a_thread_gives_the_same_bits(delta_rule):
    """Four sequences in one step are enough blocks for the walk to give a thread two value channels; one sequence alone is
    not.  A column's arithmetic does not depend on that: the rows and the states are equal bit for bit, and right."""
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(5)
    H, G, d, dv, n = 8, 4, 16, 128, 21
    C = 2 * G * d + H * dv
    ld = C + 2 * H + H * dv
    a_log = torch.randn(H, generator=g) * 0.5 if delta_rule else 0.9 + 0.09 * torch.rand(H, generator=g)
    dt_bias, norm_w, taps = torch.randn(H, generator=g) * 0.3, 1 + 0.1 * torch.randn(dv, generator=g), torch.randn(C, 1, generator=g) * 0.5
    rows = [torch.randn(n, ld, generator=g) for _ in range(4)]

    def run(which):
        lengths = [n] * len(which)
        seq, slot_t, starts = _step_arrays(lengths, list(range(len(which))))
        proj = torch.cat([rows[i] for i in which]).cuda()
        T = proj.shape[0]
        state = torch.zeros(len(which), H, d, dv, device="cuda")
        prep = torch.empty(T, ops.gated_delta_prep_width(H, G, d, dv), device="cuda")
        raw, out = torch.empty(T, H * dv, device="cuda"), torch.empty(T, H * dv, device="cuda")
        gz = proj[:, C + 2 * H:C + 2 * H + H * dv]
        if delta_rule:
            ops.gated_delta(proj, proj[:, C + H:C + 2 * H], gz, taps.cuda(), a_log.cuda(), dt_bias.cuda(), norm_w.cuda(), prep, raw, state,
                            None, out, seq, slot_t, starts, len(which), 0, C, H, G, d, dv, 1, 1e-5, decay=ops.DECAY_PER_HEAD)
        else:
            ops.gated_delta(proj, None, gz, None, a_log.cuda(), None, None, prep, raw, state,
                            None, out, seq, slot_t, starts, len(which), 0, 0, H, G, d, dv, 1, 1e-5, decay=ops.DECAY_CONSTANT, delta=False,
                            rotation=(None, None, 0, None, None))
        return out.cpu(), state.cpu()

    ops.reset_kernel_counts()
    together, states = run([0, 1, 2, 3])
    for i in range(4):
        alone, state = run([i])
        assert torch.equal(alone, together[i * n:(i + 1) * n]) and torch.equal(state[0], states[i]), i
    assert ops.kernel_counts().get("gated_delta_walk_kernel") == 5
    # and right: sequence 2 against the plain walk
    x = rows[2].double()
    if delta_rule:
        conv = plain.causal_conv_silu(x[:, :C], taps.double())
        q = plain.unit(conv[:, :G * d].reshape(n, G, d)) * d ** -0.5
        k = plain.unit(conv[:, G * d:2 * G * d].reshape(n, G, d))
        v = conv[:, 2 * G * d:].reshape(n, H, dv)
        beta = torch.sigmoid(x[:, C:C + H])
        dec = torch.exp(-torch.exp(a_log.double()) * plain.softplus(x[:, C + H:C + 2 * H] + dt_bias.double()))
        want = torch.stack([plain.delta_rule_walk(q[:, i // 2], k[:, i // 2], v[:, i], dec[:, i:i + 1].expand(-1, d), beta[:, i])
                            for i in range(H)], dim=1)
        want = plain.rms_norm(want, norm_w.double(), 1e-5).reshape(n, -1) * torch.sigmoid(x[:, C + 2 * H:C + 2 * H + H * dv])
    else:
        q = x[:, :G * d].reshape(n, G, d)
        k = x[:, G * d:2 * G * d].reshape(n, G, d) * d ** -0.5
        v = x[:, 2 * G * d:C].reshape(n, H, dv)
        want = torch.stack([plain.retention_walk(q[:, i // 2], k[:, i // 2], v[:, i], float(a_log[i])) for i in range(H)], dim=1)
        want = plain.rms_norm(want, None, 1e-5).reshape(n, -1) * torch.sigmoid(x[:, C + 2 * H:C + 2 * H + H * dv])
    assert rel_err(together[2 * n:3 * n].numpy(), want.numpy()) < 2e-5


@pytest.mark.parametrize("H, d, dv, rd", [(3, 12, 8, 8), (1, 9, 5, 0), (2, 64, 64, 64), (1, 136, 8, 20)])
def test_retention_kernels(H, d, dv, rd):
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(H * 10 + d)
    lengths, positions0 = [6, 1, 4], [0, 37, 5]
    T = sum(lengths)
    ld = (2 * H * d + 2 * H * dv + 3) // 4 * 4
    decay = [0.9 + 0.09 * i / H for i in range(H)]
    ang = torch.arange(64, dtype=torch.float64)[:, None] * torch.tensor([50.0 ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float64)[None, :] if rd else None
    cos = ang.cos().float().cuda() if rd else None
    sin = ang.sin().float().cuda() if rd else None
    state = torch.randn(4, H, d, dv, generator=g).cuda() * 0.1
    before = state.cpu().double()
    slots = [3, 1, 0]
    seq, slot_t, starts = _step_arrays(lengths, slots)
    pos = torch.tensor([p0 + i for p0, n in zip(positions0, lengths) for i in range(n)], dtype=torch.int32, device="cuda")
    proj = torch.randn(T, ld, generator=g)
    prep = torch.empty(T, ops.gated_delta_prep_width(H, H, d, dv), device="cuda")
    raw, out = torch.empty(T, H * dv, device="cuda"), torch.empty(T, H * dv, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    pd = proj.cuda()
    ops.gated_delta(pd, None, pd[:, 2 * H * d + H * dv:2 * H * d + 2 * H * dv], None, torch.tensor(decay, device="cuda"), None, None, prep, raw,
                    state, None, out, seq, slot_t, starts, 3, 0, 0, H, H, d, dv, 1, 1e-5, decay=ops.DECAY_CONSTANT, gate=ops.GATE_SILU,
                    delta=False, rotation=(cos, sin, rd, pos, status))
    assert int(status.item()) == 0
    at = 0
    for b, n in enumerate(lengths):
        x = proj[at:at + n].double()
        p = torch.arange(positions0[b], positions0[b] + n)
        q = plain.rotate_half_pairs(x[:, :H * d].reshape(n, H, d), p, rd, 50.0)
        k = plain.rotate_half_pairs(x[:, H * d:2 * H * d].reshape(n, H, d), p, rd, 50.0) * d ** -0.5
        v = x[:, 2 * H * d:2 * H * d + H * dv].reshape(n, H, dv)
        want = torch.zeros(n, H, dv, dtype=torch.float64)
        for i in range(H):
            S = before[slots[b], i].clone()
            for t in range(n):
                S = decay[i] * S + torch.outer(k[t, i], v[t, i])
                want[t, i] = S.T @ q[t, i]
            assert rel_err(state[slots[b], i].cpu().numpy(), S.numpy()) < 1e-5
        want = plain.rms_norm(want, None, 1e-5).reshape(n, -1) * plain.silu(x[:, 2 * H * d + H * dv:2 * H * d + 2 * H * dv])
        assert rel_err(out[at:at + n].cpu().numpy(), want.numpy()) < 2e-5, b
        at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, d, rd, tied", [(4, 2, 16, 6, True), (3, 1, 20, 0, True), (2, 2, 64, 64, False), (6, 3, 8, 2, True)])
def test_attention_operands_and_sink_attention_kernels(H, G, d, rd, tied, dtype):
    """Norm per head, rotation, temperature and the cache write, then the attention with a sink and an output weight, on one
    sequence of 21 tokens whose first 8 are already in the pages."""
    from carbon_engine_b200 import ops
    g = torch.Generator().manual_seed(H + d)
    n, page, dv = 21, 8, d if tied else 24
    width = (H + G) * d + (0 if tied else G * dv)
    ld = (width + 3) // 4 * 4
    proj = torch.randn(n, ld, generator=g)
    wq, wk = 1 + 0.2 * torch.randn(d, generator=g), 1 + 0.2 * torch.randn(d, generator=g)
    temp, sink = 1 + 0.3 * torch.randn(H, generator=g), torch.randn(H, generator=g) + 1.0
    ang = torch.arange(64, dtype=torch.float64)[:, None] * torch.tensor([90.0 ** (-2.0 * i / rd) for i in range(rd // 2)], dtype=torch.float64)[None, :] if rd else None
    cos, sin = (ang.cos().float().cuda(), ang.sin().float().cuda()) if rd else (None, None)
    k_pool = torch.full((6, G, page, d), float("nan"), device="cuda", dtype=dtype)
    v_pool = torch.full((6, G, page, dv), float("nan"), device="cuda", dtype=dtype)
    table = torch.tensor([[-1] * 4, [4, 1, 5, -1]], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    slot = torch.tensor([1], dtype=torch.int32, device="cuda")
    off_k, off_v = H * d, H * d if tied else (H + G) * d
    scale, out_scale = 0.7 / d ** 0.5 * 4, 0.8
    got = []
    for lo, hi in ((0, 8), (8, 21)):
        T = hi - lo
        pos = torch.arange(lo, hi, dtype=torch.int32, device="cuda")
        seq = torch.zeros(T, dtype=torch.int32, device="cuda")
        q = torch.empty(T, H * d, device="cuda", dtype=dtype)
        ops.norm_rope_kvwrite(proj[lo:hi].cuda(), q, k_pool, v_pool, wq.cuda(), wk.cuda(), temp.cuda(), cos, sin, pos, seq, slot, table,
                              status, 0, off_k, off_v, H, G, d, dv, rd, page, 1e-5)
        out = torch.empty(T, H * dv, device="cuda", dtype=dtype)
        ops.masked_attention(q, d, k_pool, v_pool, d, dv, None, out, pos, seq, slot, table, status, H, G, d, dv, page, 0, 0, scale, 0.0,
                             sinks=sink.cuda(), out_scale=out_scale)
        got.append(out.float().cpu().numpy())
    assert int(status.item()) == 0
    x = proj.double()
    p = torch.arange(n)
    qq = plain.rotate_half_pairs(plain.rms_norm(x[:, :H * d].reshape(n, H, d), wq.double(), 1e-5), p, rd, 90.0)
    kk_raw = x[:, off_k:off_k + G * d].reshape(n, G, d)
    kk = plain.rotate_half_pairs(plain.rms_norm(kk_raw, wk.double(), 1e-5), p, rd, 90.0)
    vv = kk_raw if tied else x[:, off_v:off_v + G * dv].reshape(n, G, dv)
    want = plain.sink_softmax_attention(qq, kk, vv, scale, temp.double(), sink.double()).reshape(n, -1).numpy() * out_scale
    assert rel_err(np.concatenate(got), want) < (1e-5 if dtype == torch.float32 else 3e-2)


# ---- each mechanism alone: one layer of each kind ----------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_layer_of_each_kind(tmp_path, name, dtype):
    folder = write_model(SINGLE[name], str(tmp_path / name), seed=7)
    toks = tokens_of(np.random.default_rng(5), 45, SINGLE[name]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, dtype)
    whole = h.run(toks)
    assert rel_err(whole, want) < TOL[dtype]
    one_by_one = h.run(toks, [1])
    assert rel_err(one_by_one, want) < TOL[dtype]
    if dtype == "float32":
        assert np.array_equal(whole, one_by_one)


def test_layers_outputs_one_after_another(tmp_path):
    """The residual after every layer run (a layer that runs another's weights counts), so that a fault shows where it is."""
    from carbon_engine_b200.engine.batch import StepEntry
    folder = write_model(CASES["A"], str(tmp_path / "A"))
    cfg, w = plain.read_model(folder)
    toks = tokens_of(np.random.default_rng(1), 30, cfg["vocab"])
    trace = []
    plain.forward(cfg, w, toks, trace)
    h = Harness(folder, "float32")
    rid = h.open()
    ctx, rows, commits = h.runner.prepare([StepEntry(rid, toks, [0])])
    got = []
    h.model.forward(ctx, h.storage, tap=lambda i, x: got.append(x.cpu().numpy().copy()))
    assert len(got) == len(trace) == 7
    for i, (a, b) in enumerate(zip(got, trace)):
        assert rel_err(a, b.numpy()) < 1e-4, i


# ---- whole models: cuts, batches, reuse ------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_whole_prompt_portions_and_decoding(tmp_path, name, dtype):
    from carbon_engine_b200 import ops
    folder = write_model(CASES[name], str(tmp_path / name), seed=11)
    toks = tokens_of(np.random.default_rng(3), 140 if name in ("T", "V") else 83, CASES[name]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, dtype, page_size=8, pages=24)          # 192 tokens of pages: every run reuses the last one's
    ops.reset_kernel_counts()
    whole = h.run(toks)
    if name in ("T", "V"):        # head sizes of the tensor-core kernels: bfloat16 must have taken them, float32 never
        flash = "attention_prefill_tc_kernel" if name == "T" else "attention_prefill_kernel"       # heads of 64 / of 32
        assert (flash in ops.kernel_counts()) == (dtype == "bfloat16")
    assert rel_err(whole, want) < TOL[dtype], "whole"
    for cuts in ([1], [2], [3, 2, 7, 2, 16, 5], [40, 1, 1, 1], [64, 19]):
        got = h.run(toks, cuts)
        assert rel_err(got, want) < TOL[dtype], cuts
        if dtype == "float32":
            assert np.array_equal(got, whole), cuts
    if name == "T" and dtype == "bfloat16":          # single tokens: the split-KV kernel fed by TMA, merged inside a cluster
        assert any(k.startswith("attention_decode_tma_kernel") for k in ops.kernel_counts())
    m = h.storage.manager
    assert all(m.free_pages(g) == h.storage.groups[g].num_pages for g in range(len(h.storage.groups))) and m.free_slots() == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_with_reused_pages_and_slots(tmp_path, dtype):
    """Up to three live requests, portions beside single tokens, a request left out of some steps, finished requests'
    pages and slots taken by the next: every row equals the request alone."""
    name = "A"
    folder = write_model(CASES[name], str(tmp_path / name), seed=13)
    rng = np.random.default_rng(9)
    lengths = [61, 17, 40, 1, 2, 33, 25]
    reqs = [tokens_of(rng, n, CASES[name]["vocab"]) for n in lengths]
    want = [plain_logits(folder, t) for t in reqs]
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
        assert rel_err(got, want[i]) < TOL[dtype], i
        if alone is not None:
            assert np.array_equal(got, alone[i]), i
    assert h.storage.manager.free_slots() == 3


# ---- a key that stands out, far away and at page borders; the sink ------------------------------------------------
def standout_model(tmp_path, tag, sink=None, heads=2, kv_heads=1, d=16, rot_dims=6, scale=2.0):
    """One pair layer whose attention makes EVERY query score the marker token's key far above hundreds of others.  The
    first embedding element is the same large number for every token, so the first normed element is nearly constant; one
    query element (past the rotated ones) reads it, and the same key element reads the direction of the marker's embedding:
    after the keys' norm (which a constant key element keeps alike for all tokens) it is large for the marker and noise for all others.  The delta rule beside it counts for nothing."""
    from helpers import read_raw_safetensors, write_safetensors_plain
    W, j = 32, 10
    raw = config([pair(heads=heads, kv_heads=kv_heads, dim=d, rot_dims=rot_dims, scale=scale, left_scale=1.0, right_scale=0.0)],
                 width=W, vocab=50, scale=1.0)
    folder = write_model(raw, str(tmp_path / f"standout_{tag}"), seed=21)
    path = os.path.join(folder, "model.safetensors")
    t = read_raw_safetensors(path)
    t["embed"] = (t["embed"].float() * 30.0)
    t["embed"][:, 0] = 3.0
    t["embed"] = t["embed"].to(torch.bfloat16)
    t["l0.norm1"] = torch.ones(W)
    mark = t["embed"][7].float().clone()
    mark[0] = 0.0
    mark = mark / mark.norm()
    first = torch.zeros(W); first[0] = 1.0
    for head in range(heads):
        t["l0.mix.left.q"][head * d + j] = (2.0 * first).to(t["l0.mix.left.q"].dtype)
    for head in range(kv_heads):
        t["l0.mix.left.k"][head * d + j] = (0.8 * mark).to(t["l0.mix.left.k"].dtype)
        # another key element is the same large number for every token, so that the keys' norm divides all keys alike
        t["l0.mix.left.k"][head * d + j + 1] = (2.0 * first).to(t["l0.mix.left.k"].dtype)
    # the marker's value (its projected key) is large in the same element: the output product spreads it over the residual
    sign = torch.tensor([1.0 if (3 * c) % 7 < 4 else -1.0 for c in range(W)])
    for head in range(heads):
        t["l0.mix.left.o"][:, head * d + j] = ((0.6 + 0.3 * head) * sign).to(t["l0.mix.left.o"].dtype)
    t["l0.mix.left.q.norm"], t["l0.mix.left.k.norm"] = torch.ones(d), torch.ones(d)
    t["l0.mix.left.temp"] = torch.tensor([1.0, 1.3][:heads] + [1.0] * max(0, heads - 2))
    t["l0.mix.left.sink"] = torch.full((heads,), -20.0) if sink is None else torch.tensor(sink, dtype=torch.float32)
    write_safetensors_plain(path, t)
    return folder, raw


def marker_effect(folder, toks, at):
    """How far the plain model's rows move when the marker at ``at`` is replaced by an ordinary token."""
    want = plain_logits(folder, toks)
    other = list(toks)
    other[at] = 9
    return want, np.abs(want - plain_logits(folder, other)).max(axis=1) / np.abs(want).max()


#: key sizes of the standout models with the scale that keeps the marker's score near 14: heads of 16 (in bfloat16 the
#: mma.sync flash kernel and the cp.async decode kernel) and of 64 (the tcgen05 flash kernel and the TMA decode kernel)
STANDOUT_HEADS = {16: 2.0, 64: 0.5}


@pytest.mark.parametrize("d", sorted(STANDOUT_HEADS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_and_at_page_borders(tmp_path, dtype, d):
    from carbon_engine_b200 import ops
    folder, raw = standout_model(tmp_path, "far", d=d, scale=STANDOUT_HEADS[d])
    ops.reset_kernel_counts()
    rng = np.random.default_rng(6)
    base = [int(t) for t in rng.integers(10, 50, 720)]
    h = Harness(folder, dtype, page_size=16, pages=48, max_step_tokens=1024)
    for marker_at in (3, 15, 16, 31):
        toks = list(base)
        toks[marker_at] = 7
        want, moved = marker_effect(folder, toks, marker_at)
        assert moved[marker_at:].min() > 0.1 and moved[:marker_at].max() < 1e-12          # the plain model says the far key matters
        assert rel_err(h.run(toks), want) < TOL[dtype], marker_at
        rid = h.open()
        rows = [h.step([(rid, toks[:690], [689])])]
        for p in range(690, 720):
            rows.append(h.step([(rid, toks[p:p + 1], [0])]))
        h.close(rid)
        assert rel_err(np.concatenate(rows), want[689:]) < TOL[dtype], marker_at
    if dtype == "bfloat16":
        ran = ops.kernel_counts()
        assert ("attention_prefill_tc_kernel" if d == 64 else "attention_prefill_kernel") in ran
        assert any(k.startswith("attention_decode_tma_kernel" if d == 64 else "attention_decode_kernel") for k in ran)


@pytest.mark.parametrize("d", sorted(STANDOUT_HEADS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_takes_its_share_of_every_head(tmp_path, dtype, d):
    """A sink about as large as the marker's score takes much of the marker's weight in one head and leaves the other alone; a model
    that left the sink out, scaled it or gave it the head's temperature would differ visibly."""
    folder, raw = standout_model(tmp_path, "sink", sink=[13.0, -3.0], d=d, scale=STANDOUT_HEADS[d])     # about the marker's score in head 0
    no_sink, _ = standout_model(tmp_path, "nosink", sink=[-30.0, -30.0], d=d, scale=STANDOUT_HEADS[d])
    rng = np.random.default_rng(2)
    toks = [int(t) for t in rng.integers(10, 50, 200)]
    toks[5] = 7
    want = plain_logits(folder, toks)
    assert rel_err(plain_logits(no_sink, toks), want) > 0.05            # the plain model itself: the sink matters
    h = Harness(folder, dtype, page_size=8, pages=32)
    whole = h.run(toks)
    assert rel_err(whole, want) < TOL[dtype]
    for cuts in ([1], [2], [150, 3, 1]):
        got = h.run(toks, cuts)
        assert rel_err(got, want) < TOL[dtype], cuts
        if dtype == "float32":
            assert np.array_equal(got, whole)


def test_long_decoding_keeps_the_state(tmp_path):
    """300 tokens one by one after a short prompt, in float32: the recurrent states, the convolutions' kept rows and the
    pages must carry every token (bit for bit the rows of the whole prompt)."""
    folder = write_model(CASES["C"], str(tmp_path / "C"), seed=2)
    toks = tokens_of(np.random.default_rng(8), 310, CASES["C"]["vocab"])
    want = plain_logits(folder, toks)
    h = Harness(folder, "float32", page_size=8, pages=48)
    whole = h.run(toks)
    got = h.run(toks, [10] + [1] * 300)
    assert rel_err(got, want) < TOL["float32"] and np.array_equal(got, whole)


def test_an_early_token_reaches_far_through_the_states(tmp_path):
    """With decays close to 1 a token still counts 400 tokens later, in retention and in the delta rule: the plain model
    says so, and the engine's decoded rows agree with it."""
    raw = config([retention(heads=2, dim=12, vdim=8, decay=(0.999, 0.9995), rot_dims=4, ff=None), delta(conv=2, ff=24)], scale=2.0)
    folder = write_model(raw, str(tmp_path / "far_state"), seed=4)
    rng = np.random.default_rng(10)
    toks = tokens_of(rng, 420, raw["vocab"])
    want, moved = marker_effect(folder, toks, 2)
    assert moved[400:].min() > 1e-4
    h = Harness(folder, "float32", page_size=8, pages=8, max_step_tokens=512)
    rid = h.open()
    rows = [h.step([(rid, toks[:395], [394])])] + [h.step([(rid, toks[p:p + 1], [0])]) for p in range(395, 420)]
    h.close(rid)
    assert rel_err(np.concatenate(rows), want[394:]) < TOL["float32"]


def test_first_tokens_of_a_sequence_in_a_reused_slot(tmp_path):
    """A slot and pages that held a longer request: the next request's first tokens must start from nothing (zero
    states, no kept convolution inputs, no keys), also when it is shorter than the convolution."""
    folder = write_model(CASES["A"], str(tmp_path / "A"), seed=5)
    rng = np.random.default_rng(12)
    h = Harness(folder, "float32", page_size=8, pages=12, slots=1, poison=False)
    h.run(tokens_of(rng, 90, CASES["A"]["vocab"]))
    for n in (1, 2, 3, 9):
        toks = tokens_of(rng, n, CASES["A"]["vocab"])
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


def test_trace_replay_program_on_a_pugozen_folder(tmp_path):
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


def test_command_line_writes_and_generates_a_pugozen_model(tmp_path):
    """``tiny-model --arch pugozen`` then ``generate``: the printed ids are the plain implementation's greedy ones."""
    import ast, re, subprocess, sys
    from helpers import ROOT
    carbon = [sys.executable, os.path.join(ROOT, "bin", "carbon")]
    out = str(tmp_path / "tiny_p")
    p = subprocess.run(carbon + ["tiny-model", "--arch", "pugozen", "--out", out, "--layers", "6", "--hidden", "48", "--heads", "3",
                                 "--kv-heads", "1", "--head-dim", "16", "--vocab", "120", "--seed", "9", "--shared-from", "4",
                                 "--max-positions", "256"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "wrote" in p.stdout, p.stderr[-2000:]
    cfg, w = plain.read_model(out)
    assert cfg["architecture"] == "Pugozen" and len(cfg["layers"]) == 6 and cfg["layers"][5]["weights_of"] == 1
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
