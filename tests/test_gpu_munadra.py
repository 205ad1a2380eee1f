"""The Munadra decoder through the framework's own loader, cache, step function and generation loop,
against the plain implementation (tests/plain_munadra.py), in float32 and bfloat16.

The float32 runs are the sharp ones: they differ from the plain implementation only by the order of sums,
so a key that is missed, a sink that is left out, a state that is lost or a tap that is one token off
shows at once.  The configurations are in munadra_helpers.py.
"""
from __future__ import annotations

import json

import pytest
import torch

import plain_munadra as P
from munadra_helpers import CONFIGS, assert_logits, oracle_logits, random_weights, read_folder, tokens, write_folder

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
FULL = ["mixed", "odd", "wide"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name: str, seed: int = 0, gain: float = 1.0) -> str:
        key = (name, seed, gain)
        if key not in made:
            c = CONFIGS[name]
            made[key] = write_folder(str(tmp_path_factory.mktemp(f"munadra-{name}")), c, random_weights(c, seed, gain))
        return made[key]

    return get


@pytest.fixture(scope="module")
def models(folders):
    from kuiperllama_b200.engine import load_model
    made = {}

    def get(name: str, dtype: str, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in made:
            folder = folders(name, **kw)
            with torch.inference_mode():
                made[key] = (load_model(folder, dtype=dtype, device="cuda:0"), folder)
        return made[key]

    return get


def _engine(model, max_tokens=64 * 16, use_graphs=False):
    from kuiperllama_b200.engine import Engine
    return Engine(model, model.new_cache(max_tokens=max_tokens), use_graphs=use_graphs)


def _inputs(slot, toks, want=None):
    from kuiperllama_b200.engine import SequenceInput
    return SequenceInput(slot, list(toks), list(range(len(toks))) if want is None else want)


def _run_in_steps(engine, toks, cuts):
    """One sequence fed in steps of the given sizes; logits of every token."""
    rows, at = [], 0
    with torch.inference_mode():
        slot = engine.alloc_slot()
        for n in cuts:
            rows.append(engine.step([_inputs(slot, toks[at:at + n])]).clone())
            at += n
        engine.free_slot(slot)
    assert at == len(toks)
    engine.check_device_errors()
    return torch.cat(rows)


# ----------------------------------------------------------------------------- each mechanism alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["only_latent", "only_shared", "only_rglru", "only_moe", "only_dense"])
def test_one_mechanism_alone(models, name, dtype):
    model, folder = models(name, dtype, seed=3)
    toks = tokens(70, CONFIGS[name]["vocab"], seed=11)
    ref = oracle_logits(folder, toks)
    assert_logits(_run_in_steps(_engine(model), toks, [70]), ref, dtype, f"{name}: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [1] * 70), ref, dtype, f"{name}: token by token")


@pytest.mark.parametrize("dtype", DTYPES)
def test_grouped_product_batched_and_routed(dtype):
    """The grouped product alone: per-head projections with column strides, and a routed list with padding,
    plain and with the gated activation, in tiles of 16 and of 64 rows."""
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(2)
    rnd = lambda *s: torch.randn(*s, generator=g)
    tol = 1e-5 if dtype == "float32" else 2e-2
    # batched: 5 groups read 12 of every 20 columns and write 7 of every 9
    a, w = rnd(37, 5 * 20).to(dt), (rnd(5, 7, 12) / 3).to(dt)
    for tile in (16, 64):
        out = torch.zeros(37, 5 * 9, dtype=dt, device=dev)
        ops.grouped_gemm(a.to(dev), w.to(dev), out, a_group_stride=20, out_group_stride=9, rows=37, tile_rows=tile)
        want = torch.einsum("tgk,gnk->tgn", a.double().reshape(37, 5, 20)[..., :12], w.double())
        got = out.cpu().double().reshape(37, 5, 9)
        assert torch.allclose(got[..., :7], want, atol=tol, rtol=tol) and float(got[..., 7:].abs().max()) == 0.0
        gate = rnd(37, 5).to(dt)                                           # one number per row and group on the result
        ops.grouped_gemm(a.to(dev), w.to(dev), out, a_group_stride=20, out_group_stride=9, rows=37, tile_rows=tile, row_gate=gate.to(dev))
        got = out.cpu().double().reshape(37, 5, 9)
        assert torch.allclose(got[..., :7], want * torch.sigmoid(gate.double())[..., None], atol=tol, rtol=tol)
    # batched with 16-byte aligned slices and many rows (bfloat16: the tensor-core form): 3 groups read 40 of every 48 columns
    a, w, gate = rnd(150, 3 * 48).to(dt), (rnd(3, 70, 40) / 4).to(dt), rnd(150, 3).to(dt)
    out = torch.zeros(150, 3 * 72, dtype=dt, device=dev)
    ops.grouped_gemm(a.to(dev), w.to(dev), out, a_group_stride=48, out_group_stride=72, rows=150, row_gate=gate.to(dev))
    want = torch.einsum("tgk,gnk->tgn", a.double().reshape(150, 3, 48)[..., :40], w.double()) * torch.sigmoid(gate.double())[..., None]
    got = out.cpu().double().reshape(150, 3, 72)
    assert torch.allclose(got[..., :70], want, atol=tol * 2, rtol=tol) and float(got[..., 70:].abs().max()) == 0.0
    # routed: 50 tokens choose 2 of 6 groups (one group gets nobody)
    x, wgu, choice = rnd(50, 24).to(dt), (rnd(6, 2 * 10, 24) / 4).to(dt), torch.randint(0, 5, (50, 2), generator=g).int()
    for tile in (16, 64):
        pair_pos, list_rows, tile_group = ops.moe_plan(choice.to(dev), 6, tile)
        pp, lr, tg = pair_pos.cpu(), list_rows.cpu(), tile_group.cpu()
        assert sorted(pp.tolist()) == sorted(i for i, r in enumerate(lr.tolist()) if r >= 0), "every pair has a place of its own"
        for p in range(100):
            assert lr[pp[p]] == p // 2 and tg[pp[p] // tile] == choice.reshape(-1)[p]
        for gated in (None, (0.8, 1.702, 1.0), (0.0, 1.0, 0.0)):
            N = 10 if gated else 20
            out = torch.zeros(lr.numel(), N, dtype=dt, device=dev)
            ops.grouped_gemm(x.to(dev), wgu.to(dev), out, a_rows=list_rows, tile_group=tile_group, tile_rows=tile, gated=gated)
            for p in range(0, 100, 7):
                full = wgu[choice.reshape(-1)[p]].double() @ x[p // 2].double()
                if gated:
                    gt, up = full[:10], full[10:]
                    if gated[0] > 0:
                        gt, up = gt.clamp(max=gated[0]), up.clamp(-gated[0], gated[0])
                    full = gt * torch.sigmoid(gated[1] * gt) * (up + gated[2])
                assert torch.allclose(out[pp[p]].cpu().double(), full, atol=tol, rtol=tol), (tile, gated, p)


def test_grouped_product_on_the_tensor_cores():
    """The routed product in tiles of 128 places on the tensor cores (bfloat16): experts with no rows, with a few, with
    more than a tile; plain and with the gated activation in the epilogue over interleaved gate and up rows."""
    from kuiperllama_b200.csrc import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(6)
    E, K, ff, n, top = 6, 192, 128, 330, 2
    x = torch.randn(n, K, generator=g).bfloat16()
    choice = torch.randint(0, E - 1, (n, top), generator=g).int()
    choice[:, 1] = (choice[:, 0] + 1 + choice[:, 1] % (E - 2)) % (E - 1)      # two different experts, expert E - 1 gets nobody
    choice[:3, 0] = 0
    gate, up = (torch.randn(E, ff, K, generator=g) / 8).bfloat16(), (torch.randn(E, ff, K, generator=g) / 8).bfloat16()
    down = (torch.randn(E, 72, ff, generator=g) / 8).bfloat16()
    wgu = torch.stack([ops.interleave_gate_up(gate[e], up[e]) for e in range(E)]).to(dev)
    pair_pos, list_rows, tile_group = ops.moe_plan(choice.to(dev), E, 128)
    rows = ops.moe_gather(x.to(dev), list_rows)
    lr = list_rows.cpu()
    assert torch.equal(rows.cpu()[lr >= 0], x[lr[lr >= 0].long()]) and float(rows.cpu()[lr < 0].abs().max()) == 0.0
    for gated in ((0.8, 1.702, 1.0), (0.0, 1.0, 0.0)):
        act = torch.full((lr.numel(), ff), 7.0, dtype=torch.bfloat16, device=dev)
        ops.gemm_tcgen05_grouped(rows, wgu, act, tile_group, gated=gated)
        res = torch.empty((lr.numel(), 72), dtype=torch.bfloat16, device=dev)
        ops.gemm_tcgen05_grouped(act, down.to(dev), res, tile_group)
        ops.check_status(torch.device(dev))
        pp = pair_pos.cpu()
        for p in range(0, n * top, 13):
            e, xr = int(choice.reshape(-1)[p]), x[p // top].double()
            gt, u = gate[e].double() @ xr, up[e].double() @ xr
            if gated[0] > 0:
                gt, u = gt.clamp(max=gated[0]), u.clamp(-gated[0], gated[0])
            y = gt * torch.sigmoid(gated[1] * gt) * (u + gated[2])
            assert torch.allclose(act[pp[p]].cpu().double(), y, atol=2e-2, rtol=2e-2), (gated, p)
            assert torch.allclose(res[pp[p]].cpu().double(), down[e].double() @ act[pp[p]].cpu().double(), atol=2e-2, rtol=2e-2), (gated, p)


def test_grouped_product_for_few_rows():
    """The routed product's form for a decode step (a warp per four weight rows), against the tiled form: bfloat16."""
    from kuiperllama_b200.csrc import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(16)
    E, K, ff, n, top = 7, 200, 128, 9, 3
    x = torch.randn(n, K, generator=g).bfloat16().to(dev)
    choice = torch.stack([torch.randperm(E - 1, generator=g)[:top] for _ in range(n)]).int()
    gate, up = (torch.randn(E, ff, K, generator=g) / 8).bfloat16(), (torch.randn(E, ff, K, generator=g) / 8).bfloat16()
    down = (torch.randn(E, 70, ff, generator=g) / 8).bfloat16().to(dev)
    pair_pos, list_rows, tile_group = ops.moe_plan(choice.to(dev), E, 16)
    cap = list_rows.numel()
    for inter in (False, True):
        w = torch.stack([ops.interleave_gate_up(gate[e], up[e]) if inter else torch.cat([gate[e], up[e]]) for e in range(E)]).to(dev)
        for gated in ((0.8, 1.702, 1.0), (0.0, 1.0, 0.0)):
            want, got = (torch.zeros(cap, ff, dtype=torch.bfloat16, device=dev) for _ in range(2))
            ops.grouped_gemm(x, w, want, a_rows=list_rows, tile_group=tile_group, tile_rows=16, gated=gated, interleaved=inter)
            ops.grouped_gemv(x, w, got, list_rows, tile_group, 16, gated=gated, interleaved=inter)
            assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2) and float(want.abs().max()) > 0.1
            want2, got2 = (torch.zeros(cap, 70, dtype=torch.bfloat16, device=dev) for _ in range(2))
            ops.grouped_gemm(want, down, want2, tile_group=tile_group, tile_rows=16)
            ops.grouped_gemv(want, down, got2, None, tile_group, 16, live_rows=list_rows)
            live = (list_rows >= 0)
            assert torch.allclose(got2.float()[live], want2.float()[live], atol=2e-2, rtol=2e-2)
            assert float(got2.float()[~live].abs().max()) == 0.0, "padding places are left alone"
            if inter and K % 8 == 0:
                # the same on the tensor cores, weights as tile rows
                rows = ops.moe_gather(x, list_rows)
                got3, got4 = torch.zeros_like(want), torch.zeros_like(want2)
                ops.gemm_tcgen05_grouped_skinny(rows, w, got3, tile_group, gated=gated)
                ops.gemm_tcgen05_grouped_skinny(want, down, got4, tile_group)
                ops.check_status(torch.device(dev))
                assert torch.allclose(got3.float()[live], want.float()[live], atol=2e-2, rtol=2e-2)
                assert torch.allclose(got4.float()[live], want2.float()[live], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("H, Dk, Dv", [(6, 96, 64), (32, 288, 256), (80, 48, 16), (3, 160, 144)])
def test_latent_attention_on_the_tensor_cores(H, Dk, Dv):
    """The tensor-core kernel for many heads over one key head against the plain kernel (bfloat16): prompts of unequal lengths
    on scattered pages, portions that start inside a page, single tokens; with sinks."""
    from kuiperllama_b200.csrc import ops
    from kuiperllama_b200.parts.base import StepContext
    dev = "cuda:0"
    g = torch.Generator().manual_seed(H)
    cache = (torch.randn(12, 1, 64, Dk, generator=g)).bfloat16().to(dev)
    table = torch.tensor([[5, 2, 9, 0], [1, 7, 3, 11], [4, 6, 8, 10]], dtype=torch.int32, device=dev)
    sink = torch.randn(H, generator=g).to(dev) * 2
    for starts, news in (([0, 0, 0], [130, 1, 67]), ([100, 63, 200], [30, 2, 1]), ([150, 64, 255], [1, 1, 1])):
        n = sum(news)
        q = (torch.randn(n, H * Dk, generator=g) / 4).bfloat16().to(dev)
        cu = [0]
        for k in news:
            cu.append(cu[-1] + k)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        pos = i32([st + i for st, k in zip(starts, news) for i in range(k)])
        tslot = i32([sl for sl, k in enumerate(news) for _ in range(k)])
        step = StepContext(n_tokens=n, n_seqs=3, token_ids=pos, positions=pos, token_slot=tslot, seq_slots=i32([0, 1, 2]), seq_starts=i32(starts),
                           seq_new=i32(news), cu_tokens=i32(cu), is_decode=max(news) == 1, max_new=max(news), max_context=max(a + b for a, b in zip(starts, news)),
                           host_slots=[0, 1, 2], host_starts=starts, host_new=news)
        step.context_class = 1 if max(news) == 1 and H == 6 else 0           # a decode step: another number of pieces
        for sk in (None, sink):
            want = torch.empty(n, H * Dv, dtype=torch.bfloat16, device=dev)
            got = torch.full_like(want, 9.0)
            ops.attention_simt(q, H * Dk, want, cache, cache, table, pos, tslot, n, H, 1, Dk, 0.3, 0, value_dim=Dv, sink=sk)
            ops.latent_attention(q, got, cache, table, step, H, Dk, Dv, 0.3, sk)
            assert torch.allclose(got.float(), want.float(), atol=3e-2, rtol=3e-2), (starts, news, sk is not None)


def test_router_softmax_top_and_weights():
    """Scores over all experts, the largest first, the lower index among equals, weights not renormalised (or renormalised)."""
    from kuiperllama_b200.csrc import ops
    g = torch.Generator().manual_seed(4)
    for E, top in ((16, 4), (7, 7), (3, 1), (40, 33), (200, 5)):
        z = torch.randn(29, E, generator=g) * 2
        z[3, :] = 0.25                                                     # all equal: the first `top` experts
        choice, weight = ops.moe_route(z.cuda(), top)
        s = torch.softmax(z.double(), dim=-1)
        w_ref, i_ref = torch.topk(s, top, dim=-1)
        rows = [r for r in range(29) if r != 3]
        assert torch.equal(choice.cpu()[rows].long(), i_ref[rows])
        assert torch.allclose(weight.cpu().double(), w_ref, atol=1e-6, rtol=1e-5)
        assert choice.cpu()[3].tolist() == list(range(top))
        _, renorm = ops.moe_route(z.cuda(), top, True)
        assert torch.allclose(renorm.cpu().double(), w_ref / w_ref.sum(-1, keepdim=True), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_sink_and_value_columns(dtype):
    """The attention kernel's two options alone: values that are the first columns of the keys' rows, and a sink
    in the denominator (a large sink takes nearly all the weight: the result shrinks by that share)."""
    from kuiperllama_b200.csrc import ops
    dt, dev = getattr(torch, dtype), "cuda:0"
    g = torch.Generator().manual_seed(8)
    H, Dk, Dv, T = 3, 20, 12, 150
    rows = (torch.randn(T, Dk, generator=g)).to(dt)
    q = (torch.randn(T, H, Dk, generator=g)).to(dt)
    cache = torch.zeros(4, 1, 64, Dk, dtype=dt, device=dev)
    table = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=dev)
    for p in range(T):
        cache[int(table[0, p // 64]), 0, p % 64] = rows[p].to(dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    for sink in (None, torch.tensor([-1.0, 0.5, 9.0])):
        out = torch.empty(T, H * Dv, dtype=dt, device=dev)
        ops.attention_simt(q.reshape(T, -1).to(dev), H * Dk, out, cache, cache, table, pos, slot, T, H, 1, Dk, 0.4, 0,
                           value_dim=Dv, sink=None if sink is None else sink.to(dev))
        s = torch.einsum("ihd,jd->hij", q.double(), rows.double()) * 0.4
        s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril()[None], -float("inf"))
        e = torch.exp(s - s.max(-1, keepdim=True).values)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink.double()[:, None, None] - s.max(-1, keepdim=True).values)
        want = torch.einsum("hij,jd->ihd", e / den, rows.double()[:, :Dv])
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert torch.allclose(out.cpu().double().reshape(T, H, Dv), want, atol=tol, rtol=tol)


# ----------------------------------------------------------------------------- cuts, batches, reuse

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", FULL)
def test_whole_prompt_portions_and_single_tokens(models, name, dtype):
    model, folder = models(name, dtype, seed=1)
    toks = tokens(150, CONFIGS[name]["vocab"], seed=21)
    ref = oracle_logits(folder, toks)
    for cuts in ([150], [118] + [1] * 32, [2] * 75, [63, 1, 2, 62, 3, 1, 1, 17], [1, 64, 64, 21], [5, 59, 2, 84]):
        assert sum(cuts) == 150
        assert_logits(_run_in_steps(_engine(model), toks, cuts), ref, dtype, f"{name}: steps of {cuts[:6]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_long_prompts_take_the_chunked_scan(models, name, dtype):
    """From 256 tokens of a sequence in one step the recurrence runs in chunks of 64 side by side: a long prompt, a long
    portion after a short one and before one, and a long prompt beside a short one in one step."""
    from kuiperllama_b200.csrc import ops
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    toks = tokens(330, V, seed=41)
    assert 330 >= ops.LINEAR_SCAN_CHUNKED_FROM and 330 % ops.LINEAR_SCAN_CHUNK
    ref = oracle_logits(folder, toks)
    for cuts in ([330], [300, 30], [31, 299]):
        assert_logits(_run_in_steps(_engine(model), toks, cuts), ref, dtype, f"{name}: long steps of {cuts}")
    short = tokens(70, V, seed=42)
    eng = _engine(model)
    with torch.inference_mode():
        a, b = eng.alloc_slot(), eng.alloc_slot()
        out = eng.step([_inputs(a, short), _inputs(b, toks)])
    eng.check_device_errors()
    assert_logits(out[:70], oracle_logits(folder, short), dtype, f"{name}: a short prompt beside a long one")
    assert_logits(out[70:], ref, dtype, f"{name}: a long prompt beside a short one")


@pytest.mark.parametrize("use_graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", FULL)
def test_unequal_batches_against_each_alone(models, name, dtype, use_graphs):
    """Requests of 1 to 130 tokens in one step, then decoded together, the shorter ones leaving first."""
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    lens, more = [1, 3, 70, 130, 64], [2, 9, 5, 9, 7]
    seqs = [tokens(n + m, V, seed=30 + i) for i, (n, m) in enumerate(zip(lens, more))]
    refs = [oracle_logits(folder, s) for s in seqs]
    eng = _engine(model, max_tokens=64 * 12, use_graphs=use_graphs)
    with torch.inference_mode():
        slots = [eng.alloc_slot() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([_inputs(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
        at = 0
        for i, n in enumerate(lens):
            got[i].append(out[at:at + n].clone())
            at += n
        for k in range(max(more)):
            live = [i for i in range(len(seqs)) if k < more[i]]
            if use_graphs:
                out = eng.decode_step([slots[i] for i in live], [seqs[i][lens[i] + k] for i in live]).clone()
            else:
                out = eng.step([_inputs(slots[i], [seqs[i][lens[i] + k]]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1].clone())
            for i in live:
                if k + 1 == more[i]:
                    eng.free_slot(slots[i])
    eng.check_device_errors()
    for i in range(len(seqs)):
        assert_logits(torch.cat(got[i]), refs[i], dtype, f"{name}: request {i} of the batch")
    assert eng.cache.slots.held() == 0 and all(h == 0 for h in eng.cache.pages_held())


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_are_reused(models, dtype):
    """A cache with room for little: four rounds of requests on the same slots and pages, whose old contents
    (latent rows, recurrent state, convolution inputs) must not leak into the next request."""
    model, folder = models("mixed", dtype, seed=1)
    V = CONFIGS["mixed"]["vocab"]
    eng = _engine(model, max_tokens=64 * 5)
    for rnd in range(4):
        lens = [[100, 70], [3, 129], [64, 65], [1, 2]][rnd]
        seqs = [tokens(n + 3, V, seed=50 + 10 * rnd + i) for i, n in enumerate(lens)]
        with torch.inference_mode():
            slots = [eng.alloc_slot() for _ in seqs]
            first = eng.step([_inputs(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
            rest = [eng.step([_inputs(sl, [s[n + k]]) for sl, s, n in zip(slots, seqs, lens)]).clone() for k in range(3)]
            for sl in slots:
                eng.free_slot(sl)
        at = 0
        for i, (s, n) in enumerate(zip(seqs, lens)):
            got = torch.cat([first[at:at + n]] + [r[i:i + 1] for r in rest])
            at += n
            assert_logits(got, oracle_logits(folder, s), dtype, f"round {rnd}, request {i}")
    eng.check_device_errors()


# ----------------------------------------------------------------------------- what random weights would hide

def _needle_folder(tmp_path_factory, places, T):
    """One attention layer whose weights are made so that chosen queries read single keys far back: every head's
    unrotated query is beta * (its key map) * (the latent's map) * R with a rotation R of the model's width, the
    rotated query part is zero, and the embedding of the query token A_i is R^T times that of the needle
    token B_i; so the query of A_i scores highest on the key of B_i, wherever it lies."""
    c = json.loads(json.dumps(CONFIGS["sharp"]))
    c["layers"] = [dict(c["layers"][0])]
    c["embedding"]["scale"] = 1.0
    W = {k: v.float() for k, v in random_weights(c, 9).items()}
    m = c["layers"][0]["mixer"]
    H, d, rd, r, width = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"], c["width"]
    g = torch.Generator().manual_seed(12)
    R = torch.linalg.qr(torch.randn(width, width, generator=g, dtype=torch.float64)).Q
    A, wn, U = W["l0.mix.dkv"][:r].double(), W["l0.mix.dkv.norm"].double(), W["l0.mix.uk"].double().reshape(H, d, r)
    q = torch.zeros(H, d + rd, width, dtype=torch.float64)
    q[:, :d] = 1.5 * torch.einsum("hdr,rw->hdw", U * wn, A) @ R
    W["l0.mix.q"] = q.reshape(H * (d + rd), width).float()
    W["l0.mix.sink"] = torch.tensor([0.0, 12.0, 16.0])
    V = c["vocab"]
    toks = tokens(T, V - 2 * len(places), seed=80)                       # the last ids of the vocabulary are kept for the pairs
    for i, place in enumerate(places):
        a, b = V - 1 - 2 * i, V - 2 - 2 * i
        W["embed"][a] = (R.T @ W["embed"][b].double()).float()
        toks[place] = b
        toks[T - 1 - 2 * i] = a                                          # the queries: every other one of the last rows
    W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    return write_folder(str(tmp_path_factory.mktemp("munadra-needle")), c, W), toks


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_page_borders_and_the_sink_show(tmp_path_factory, dtype):
    """Queries that read one key each: four pages back, and at the last and first place of every page between.
    The plain implementation first proves it (the weight on that key, and that the sink takes a share); then
    prompt, portions that end on and next to page borders, and decoding across them."""
    from kuiperllama_b200.engine import load_model
    places, T = [0, 63, 64, 127, 128, 191, 192, 255, 256], 290
    folder, toks = _needle_folder(tmp_path_factory, places, T)
    c, W = read_folder(folder)
    x = W["embed"].double()[torch.tensor(toks)]
    w, _, _ = P.latent_attention_weights(x, W, "l0.mix.", c["layers"][0]["mixer"], c["norm"]["eps"])
    for i, place in enumerate(places):
        assert float(w[:, T - 1 - 2 * i, place].max()) > 0.5, f"no head of the query for place {place} reads it"
    share = 1.0 - w.sum(-1)                                              # what the sink takes, [H, T]
    assert float(share[2].median()) > 10 * float(share[0].median()) > 0, "the sinks do not differ in what they take"
    ref = oracle_logits(folder, toks)
    with torch.inference_mode():
        model = load_model(folder, dtype=dtype, device="cuda:0")
    assert_logits(_run_in_steps(_engine(model), toks, [T]), ref, dtype, "needle: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [64, 63, 1, 65, 62, 15, 20]), ref, dtype, "needle: portions at page borders")
    assert_logits(_run_in_steps(_engine(model), toks, [250] + [1] * 40), ref, dtype, "needle: prompt, then the queries one by one")
    assert_logits(_run_in_steps(_engine(model), toks, [120] + [1] * 170), ref, dtype, "needle: decoding over three borders")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_the_first_tokens_of_a_sequence(models, name, dtype):
    """Prompts shorter than the convolution's taps, a prompt of one token, and what follows token by token:
    the state starts at zero, the first token takes no other path, and taps before the start read zeros."""
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    for n in (1, 2, 3, 4):
        toks = tokens(n + 8, V, seed=60 + n)
        assert_logits(_run_in_steps(_engine(model), toks, [n] + [1] * 8), oracle_logits(folder, toks), dtype, f"{name}: prompt of {n}")
        assert_logits(_run_in_steps(_engine(model), toks, [n, 2, 2, 4]), oracle_logits(folder, toks), dtype, f"{name}: prompt of {n}, portions")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_graphs(models, dtype):
    """400 tokens one by one through captured decode steps after a prompt of five: the recurrent state and
    the latent rows over six pages."""
    model, folder = models("mixed", dtype, seed=1)
    toks = tokens(405, CONFIGS["mixed"]["vocab"], seed=70)
    eng = _engine(model, max_tokens=64 * 8, use_graphs=True)
    with torch.inference_mode():
        slot = eng.alloc_slot()
        rows = [eng.step([_inputs(slot, toks[:5])]).clone()]
        for t in toks[5:]:
            rows.append(eng.decode_step([slot], [t]).clone())
        eng.free_slot(slot)
    eng.check_device_errors()
    assert_logits(torch.cat(rows), oracle_logits(folder, toks), dtype, "long decoding")


# ----------------------------------------------------------------------------- the entry points

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    """``load(...).generate``: scheduler, batches that reuse slots, captured decode steps, sampler.  float32 gives
    the plain greedy tokens (where the plain logits' two best are apart); in bfloat16 a token may differ where
    they are close, and the run is compared up to there."""
    import kuiperllama_b200 as kl
    folder = folders(name, seed=1)
    c, W = read_folder(folder)
    prompts = [tokens(n, c["vocab"], seed=90 + n) for n in (7, 1, 66, 20, 3)]
    m = kl.load(folder, dtype=dtype, device="cuda:0", max_tokens=64 * 8, max_batch=2)
    got = m.generate(prompts, max_new_tokens=10, stop_ids=[])
    for p, out in zip(prompts, got):
        assert len(out) == 10
        seq = list(p)
        for tok in out:
            logits = P.forward(c, W, seq)[-1]
            top = torch.topk(logits, 2).values
            if int(logits.argmax()) != tok:
                close = float(top[0] - top[1]) < (1e-3 if dtype == "float32" else 0.15) * float(logits.std())
                assert close and float(logits[tok]) >= float(top[1]) - 1e-9, f"{name} {dtype}: token {tok} is not the plain greedy token"
                break
            seq.append(tok)


def test_cli_runs_a_munadra_folder(folders, capsys):
    from kuiperllama_b200.cli import main
    folder = folders("mixed", seed=1)
    assert main([folder, "--prompt-ids", "1,2,3", "--max-new-tokens", "4", "--dtype", "float32", "--stop-ids", ""]) == 0
    out = capsys.readouterr().out
    c, W = read_folder(folder)
    seq = [1, 2, 3]
    for _ in range(4):
        seq.append(int(P.forward(c, W, seq)[-1].argmax()))
    assert " ".join(str(t) for t in seq[3:]) in out


def test_trace_run_replays_a_munadra_folder(folders, tmp_path):
    """bin/trace_run as a user runs it, in float32: five requests in one step, then two steps of a token each
    with the shortest leaving first."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = folders("mixed", seed=1)
    V = CONFIGS["mixed"]["vocab"]
    lens = [1, 3, 65, 2, 66]
    seqs = [tokens(n + 2, V, seed=110 + i) for i, n in enumerate(lens)]
    steps = [{"step": 0, "entries": [{"id": f"r{i}", "tokens": s[:n], "want": [n - 1]} for i, (s, n) in enumerate(zip(seqs, lens))], "end": []},
             {"step": 1, "entries": [{"id": f"r{i}", "tokens": [s[n]], "want": [0]} for i, (s, n) in enumerate(zip(seqs, lens))], "end": ["r0"]},
             {"step": 2, "entries": [{"id": f"r{i}", "tokens": [s[n + 1]], "want": [0]} for i, (s, n) in enumerate(zip(seqs, lens)) if i],
              "end": [f"r{i}" for i in range(1, 5)]}]
    out = str(tmp_path / "out")
    cmd = [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out,
           "--max-tokens", str(sum(lens) + 2 * len(lens))]
    p = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    refs = [oracle_logits(folder, s) for s in seqs]
    read = lambda k: torch.from_numpy(np.fromfile(os.path.join(out, f"{k}.f32"), dtype="<f4").reshape(-1, V).copy())
    assert_logits(read(0), torch.stack([r[n - 1] for r, n in zip(refs, lens)]), "float32", "replay: prompts")
    assert_logits(read(1), torch.stack([r[n] for r, n in zip(refs, lens)]), "float32", "replay: first tokens")
    assert_logits(read(2), torch.stack([r[n + 1] for r, n in list(zip(refs, lens))[1:]]), "float32", "replay: second tokens")
