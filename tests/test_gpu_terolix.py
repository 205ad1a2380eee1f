"""The Terolix decoder through the framework's own loader, cache, step function and generation
loop, against the plain implementation (tests/plain_terolix.py), in float32 and bfloat16.

The float32 runs are the sharp ones: they differ from the oracle only by the order of sums, so a
key that is missed, a state that is lost or a tap that is one token off shows at once.  The
configurations are in terolix_helpers.py.
"""
from __future__ import annotations

import math

import pytest
import torch

import plain_terolix as P
from terolix_helpers import CONFIGS, assert_logits, oracle_logits, random_weights, tokens, write_folder

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
FULL = ["mixed", "odd", "wide"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name: str, seed: int = 0, gain: float = 1.0, weights=None, config=None) -> str:
        key = (name, seed, gain)
        if key not in made:
            c = config or CONFIGS[name]
            made[key] = write_folder(str(tmp_path_factory.mktemp(f"terolix-{name}")), c, weights or random_weights(c, seed, gain))
        return made[key]

    return get


@pytest.fixture(scope="module")
def models(folders):
    from kuiperllama_b200.engine import load_model
    made = {}

    def get(name: str, dtype: str, **kw):
        key = (name, dtype, tuple(sorted((k, v) for k, v in kw.items() if k in ("seed", "gain"))))
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
@pytest.mark.parametrize("name", ["only_mingru", "only_attention", "only_delta", "only_ff"])
def test_one_mechanism_alone(models, name, dtype):
    """A model of a single layer with a single sublayer of interest, whole prompt and token by token."""
    model, folder = models(name, dtype, seed=3)
    toks = tokens(70, CONFIGS[name]["vocab"], seed=11)
    ref = oracle_logits(folder, toks)
    assert_logits(_run_in_steps(_engine(model), toks, [70]), ref, dtype, f"{name}: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [1] * 70), ref, dtype, f"{name}: token by token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hid", [100, 99, 1536])
def test_norm_chain_against_the_plain_functions(dtype, hid):
    """gate, norm after, 32-bit sum, norm before, as one kernel: rows on 16-byte boundaries (the form that
    keeps a row in registers), rows on none (hid 99), the result given as rows or as float32 pieces."""
    from kuiperllama_b200.csrc import ops
    dt = getattr(torch, dtype)
    dev = "cuda:0"
    g = torch.Generator().manual_seed(5)
    n = 37
    rnd = lambda *s: torch.randn(*s, generator=g)
    x, d, gate = rnd(n, hid) * 3, rnd(n, hid).to(dt), rnd(n, hid).to(dt)
    gb, pw, pb, w, b = rnd(hid), 1 + 0.3 * rnd(hid), rnd(hid), 1 + 0.3 * rnd(hid), rnd(hid)
    tol = 1e-5 if dtype == "float32" else 2e-2
    for kind in ("layernorm", "rmsnorm"):
        def norm(t, ww, bb, eps):
            return P.layer_norm(t, ww, bb, eps) if kind == "layernorm" else P.rms_divide(t, eps) * ww + bb
        want_x = x.double() + norm(d.double() * P.sigmoid(gate.double() + gb.double()), pw.double(), pb.double(), 1e-5)
        want = norm(want_x, w.double(), b.double(), 2e-6)
        res, out = x.to(dev).clone(), torch.empty(n, hid, dtype=dt, device=dev)
        wide = torch.cat([gate, d], dim=1).to(dev)                      # both as column slices of one matrix
        ops.norm_chain(res, wide[:, hid:], out, w.to(dev), b.to(dev), 2e-6, kind, gate=wide[:, :hid], gate_bias=gb.to(dev),
                       post=(pw.to(dev), pb.to(dev), 1e-5, kind))
        assert torch.allclose(res.cpu().double(), want_x, atol=1e-5, rtol=1e-5), kind
        assert torch.allclose(out.cpu().double(), want, atol=tol * 4, rtol=tol), kind
        rows = torch.tensor([5, 0, 36], dtype=torch.int32, device=dev)
        res2, out2 = x.to(dev).clone(), torch.empty(3, hid, dtype=dt, device=dev)
        ops.norm_chain(res2, wide[:, hid:], out2, w.to(dev), b.to(dev), 2e-6, kind, gate=wide[:, :hid], gate_bias=gb.to(dev),
                       post=(pw.to(dev), pb.to(dev), 1e-5, kind), rows=rows)
        assert torch.equal(res2.cpu(), x), "with rows the stream stays as it is"
        assert torch.equal(out2, out[rows.long()])
        # the same result handed over as three float32 pieces
        pieces = torch.stack([d.float() * 0.5, d.float() * 0.25, d.float() * 0.25]).to(dev).contiguous()
        res3, out3 = x.to(dev).clone(), torch.empty(n, hid, dtype=dt, device=dev)
        ops.norm_chain(res3, pieces, out3, w.to(dev), b.to(dev), 2e-6, kind, gate=wide[:, :hid], gate_bias=gb.to(dev),
                       post=(pw.to(dev), pb.to(dev), 1e-5, kind))
        assert torch.allclose(res3, res, atol=1e-5, rtol=1e-5) and torch.allclose(out3.float(), out.float(), atol=tol, rtol=tol)
        # nothing to add: the norm of the stream alone; and the sum alone
        res4, out4 = x.to(dev).clone(), torch.empty(n, hid, dtype=dt, device=dev)
        ops.norm_chain(res4, None, out4, w.to(dev), b.to(dev), 2e-6, kind)
        assert torch.equal(res4.cpu(), x) and torch.allclose(out4.cpu().double(), norm(x.double(), w.double(), b.double(), 2e-6), atol=tol * 4, rtol=tol)
        ops.norm_chain(res4, wide[:, hid:], None, None, None, 0.0, kind)
        assert torch.allclose(res4.cpu().double(), x.double() + d.double(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_kernels_against_the_plain_functions(dtype):
    """The other new kernels one by one on random inputs: activations, the sigmoid gate, the per-head norm."""
    from kuiperllama_b200.csrc import ops
    dt = getattr(torch, dtype)
    dev = "cuda:0"
    g = torch.Generator().manual_seed(6)
    n, hid = 37, 100
    rnd = lambda *s: torch.randn(*s, generator=g)
    tol = 1e-5 if dtype == "float32" else 2e-2
    z = (rnd(n, hid) * 2).to(dt)
    params = torch.tensor([float(P.softplus(torch.tensor(0.3, dtype=P.F))), 0.5 + float(P.softplus(torch.tensor(-0.7, dtype=P.F)))])
    got = torch.empty(n, hid, dtype=dt, device=dev)
    ops.activation(z.to(dev), got, "xielu", params.to(dev))
    assert torch.allclose(got.cpu().double(), P.xielu(z.double(), 0.3, -0.7), atol=tol, rtol=tol)
    odd = torch.empty(n, hid - 1, dtype=dt, device=dev)                 # a width that takes the element-by-element form
    ops.activation(z.to(dev)[:, 1:], odd, "xielu", params.to(dev))
    assert torch.equal(odd, got[:, 1:])
    ops.activation(z.to(dev), got, "gelu_tanh")
    zz = z.double()
    assert torch.allclose(got.cpu().double(), 0.5 * zz * (1 + torch.tanh(math.sqrt(2 / math.pi) * (zz + 0.044715 * zz ** 3))), atol=tol, rtol=tol)
    y = rnd(n, hid).to(dt).to(dev)
    want = y.cpu().double() * P.sigmoid(z.double())
    ops.sigmoid_gate(y, z.to(dev))
    assert torch.allclose(y.cpu().double(), want, atol=tol, rtol=tol)
    heads, dim = 5, 20
    o, hw = rnd(n, heads * dim).to(dev), (1 + 0.3 * rnd(dim))
    want = (P.rms_divide(o.cpu().double().view(n, heads, dim), 1e-5) * hw.double()).reshape(n, hid) * P.silu(z.double())
    got = torch.empty(n, hid, dtype=dt, device=dev)
    ops.head_rmsnorm_gate(o, z.to(dev), hw.to(dev), got, heads, dim, 1e-5)
    assert torch.allclose(got.cpu().double(), want, atol=tol * 2, rtol=tol)


# ----------------------------------------------------------------------------- whole models, cut in every way

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", FULL + ["grouped"])
def test_whole_prompt_and_token_by_token(models, name, dtype):
    """150 tokens at once (keys in three pages), and the same one by one from the first token on."""
    model, folder = models(name, dtype, seed=1)
    toks = tokens(150, CONFIGS[name]["vocab"], seed=21)
    ref = oracle_logits(folder, toks)
    assert_logits(_run_in_steps(_engine(model), toks, [150]), ref, dtype, f"{name}: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [1] * 150), ref, dtype, f"{name}: token by token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", FULL)
@pytest.mark.parametrize("cuts", [[63, 2, 64, 1, 20], [2, 2, 3, 57, 1, 70, 15], [1, 128, 21]])
def test_portions(models, name, dtype, cuts):
    """A prompt in portions down to two tokens and one, ending at, just before and just after page
    borders; every portion starts from the state, taps and keys that the one before left."""
    model, folder = models(name, dtype, seed=1)
    toks = tokens(sum(cuts), CONFIGS[name]["vocab"], seed=22)
    assert_logits(_run_in_steps(_engine(model), toks, cuts), oracle_logits(folder, toks), dtype, f"{name}: portions {cuts}")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_unequal_batch_then_decoding_together(models, name, dtype, graphs):
    """Prompts of 1, 2, 5, 64, 65 and 130 tokens in one step, then 40 steps of one token each; the
    short ones end earlier.  Every row equals what its sequence gives alone.  With graphs the steps
    are the captured ones that generation uses (padded rows included)."""
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    lens, tails = [1, 2, 5, 64, 65, 130], [40, 3, 40, 17, 40, 40]
    seqs = [tokens(n + t, V, seed=30 + i) for i, (n, t) in enumerate(zip(lens, tails))]
    refs = [oracle_logits(folder, s) for s in seqs]
    engine = _engine(model, max_tokens=64 * 24, use_graphs=graphs)
    with torch.inference_mode():
        slots = [engine.alloc_slot() for _ in seqs]
        got = engine.step([_inputs(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
        assert_logits(got, torch.cat([r[:n] for r, n in zip(refs, lens)]), dtype, f"{name}: the step of all prompts")
        for j in range(max(tails)):
            live = [i for i in range(len(seqs)) if j < tails[i]]
            if graphs:
                got = engine.decode_step([slots[i] for i in live], [seqs[i][lens[i] + j] for i in live]).clone()
            else:
                got = engine.step([_inputs(slots[i], [seqs[i][lens[i] + j]]) for i in live])
            assert_logits(got, torch.stack([refs[i][lens[i] + j] for i in live]), dtype, f"{name}: decode step {j}")
            for i in range(len(seqs)):
                if j + 1 == tails[i]:
                    engine.free_slot(slots[i])
    engine.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(models, dtype):
    """A cache of three slots' worth: sequences come and go, each new one lands in a slot and on pages
    that still hold an older one's state, taps and keys, and must not see them."""
    name = "mixed"
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    engine = _engine(model, max_tokens=64 * 6)
    with torch.inference_mode():
        for round_ in range(4):
            seqs = [tokens(n, V, seed=50 + 10 * round_ + i) for i, n in enumerate((90 + round_, 3, 70))]
            slots = [engine.alloc_slot() for _ in seqs]
            got = engine.step([_inputs(sl, s[:-2]) for sl, s in zip(slots, seqs)])
            assert_logits(got, torch.cat([oracle_logits(folder, s)[:-2] for s in seqs]), dtype, f"round {round_}: prompts")
            for j in (-2, -1):
                got = engine.step([_inputs(sl, [s[j]]) for sl, s in zip(slots, seqs)])
                assert_logits(got, torch.stack([oracle_logits(folder, s)[j] for s in seqs]), dtype, f"round {round_}: token {j}")
            for sl in reversed(slots):
                engine.free_slot(sl)
    engine.check_device_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [1, 2, 3, 4, 5])
def test_first_tokens(models, dtype, n):
    """Prompts shorter than the convolutions' taps (5 and 3 here) and than anything else."""
    for name in ("odd", "mixed"):
        model, folder = models(name, dtype, seed=1)
        toks = tokens(n + 2, CONFIGS[name]["vocab"], seed=60 + n)
        assert_logits(_run_in_steps(_engine(model), toks, [n, 1, 1]), oracle_logits(folder, toks), dtype, f"{name}: {n} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(models, dtype):
    """Three tokens of prompt and 400 decoded: the recurrent states run for 400 steps, the keys fill
    seven pages."""
    name = "mixed"
    model, folder = models(name, dtype, seed=1)
    toks = tokens(403, CONFIGS[name]["vocab"], seed=70)
    got = _run_in_steps(_engine(model), toks, [3] + [1] * 400)
    assert_logits(got, oracle_logits(folder, toks), dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_prompts_in_one_step(models, name, dtype):
    """Prompts of 300, 257, 256 and 70 tokens in one step (from 256 tokens on the minGRU runs chunk by
    chunk in three passes; the last chunks are part full, one sequence has a single whole chunk more
    than the threshold), then a portion of 259 more for the first, then a token each."""
    model, folder = models(name, dtype, seed=1)
    V = CONFIGS[name]["vocab"]
    seqs = [tokens(n, V, seed=75 + i) for i, n in enumerate((300 + 259 + 1, 257 + 1, 256 + 1, 70 + 1))]
    lens = [300, 257, 256, 70]
    refs = [oracle_logits(folder, s) for s in seqs]
    engine = _engine(model, max_tokens=64 * 24)
    with torch.inference_mode():
        slots = [engine.alloc_slot() for _ in seqs]
        got = engine.step([_inputs(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
        assert_logits(got, torch.cat([r[:n] for r, n in zip(refs, lens)]), dtype, f"{name}: long prompts")
        got = engine.step([_inputs(slots[0], seqs[0][300:559])])
        assert_logits(got, refs[0][300:559], dtype, f"{name}: a long portion")
        got = engine.step([_inputs(sl, [s[-1]]) for sl, s in zip(slots, seqs)])
        assert_logits(got, torch.stack([r[-1] for r in refs]), dtype, f"{name}: the tokens after")
    engine.check_device_errors()


# ----------------------------------------------------------------------------- a far key that matters

def _needle_model(folders, models, dtype):
    """One attention layer (4 heads on 2 key heads, 16 of 32 dimensions rotated) whose queries and keys
    are scaled up until every query's weights sit on one or two keys, wherever they are."""
    c = {"architecture": "Terolix", "vocab": 53, "width": 64, "norm": {"eps": 1e-5},
         "layers": [dict(CONFIGS["mixed"]["layers"][1], mlp=None)]}
    w = random_weights(c, seed=9)
    w["l0.mix.q"] = (w["l0.mix.q"].float() * 6).to(torch.bfloat16)
    w["l0.mix.k"] = (w["l0.mix.k"].float() * 6).to(torch.bfloat16)
    CONFIGS["needle"] = c
    return models("needle", dtype, weights=w, config=c)


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_matter(folders, models, dtype):
    """With sharp attention a query's answer is one far key's value: the test first makes sure (from the
    plain implementation's weights) that queries exist whose best key lies more than two pages back, in
    the page before, at a page's last and first place, then compares prompt and decoding."""
    model, folder = _needle_model(folders, models, dtype)
    c = CONFIGS["needle"]
    toks = tokens(260, c["vocab"], seed=80)
    w = P.read_weights(folder)
    x = w["embed"][torch.tensor(toks)]
    h = P.layer_norm(x, w["l0.norm1"], w["l0.norm1.b"], c["norm"]["eps"])
    probs = P.attention_weights(h, w, "l0.", c["layers"][0]["mixer"])             # [H, T, T]
    best, arg = probs.max(dim=-1)
    sharp = best > 0.5
    dist = torch.arange(260)[None, :] - arg
    assert int((sharp & (dist > 128)).sum()) >= 5, "no query reads a key more than two pages back"
    assert int((sharp & (arg % 64 == 63) & (dist > 0)).sum()) >= 1 and int((sharp & (arg % 64 == 0) & (dist > 0)).sum()) >= 1
    ref = oracle_logits(folder, toks)
    assert_logits(_run_in_steps(_engine(model), toks, [260]), ref, dtype, "needle: whole")
    assert_logits(_run_in_steps(_engine(model), toks, [190] + [1] * 70), ref, dtype, "needle: prompt, then decoding")
    assert_logits(_run_in_steps(_engine(model), toks, [100, 92, 68]), ref, dtype, "needle: portions")


# ----------------------------------------------------------------------------- the entry point

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    """``load(...).generate``: scheduler, batches that reuse slots, captured decode steps, sampler.
    float32 gives the plain greedy tokens (where the plain logits' two best are apart); in bfloat16 a
    token may differ where they are close, and the run is compared up to there."""
    import kuiperllama_b200 as kl
    folder = folders(name, seed=1)
    V = CONFIGS[name]["vocab"]
    prompts = [tokens(n, V, seed=90 + n) for n in (7, 1, 66, 20, 3)]
    m = kl.load(folder, dtype=dtype, device="cuda:0", max_tokens=64 * 8, max_batch=2)
    got = m.generate(prompts, max_new_tokens=12, stop_ids=[])
    w, c = P.read_weights(folder), P.read_config(folder)
    for p, out in zip(prompts, got):
        assert len(out) == 12
        seq = list(p)
        for tok in out:
            logits = P.forward_logits(w, c, seq)[-1]
            top = torch.topk(logits, 2).values
            spread = float(logits.std())
            if int(logits.argmax()) != tok:
                close = float(top[0] - top[1]) < (1e-3 if dtype == "float32" else 0.15) * spread
                assert close and float(logits[tok]) >= float(top[1]) - 1e-9, f"{name} {dtype}: token {tok} is not the plain greedy token"
                break
            seq.append(tok)


def test_cli_runs_a_terolix_folder(folders, capsys):
    from kuiperllama_b200.cli import main
    folder = folders("mixed", seed=1)
    assert main([folder, "--prompt-ids", "1,2,3", "--max-new-tokens", "4", "--dtype", "float32", "--stop-ids", ""]) == 0
    out = capsys.readouterr().out
    w, c = P.read_weights(folder), P.read_config(folder)
    seq = [1, 2, 3]
    for _ in range(4):
        seq.append(int(P.forward_logits(w, c, seq)[-1].argmax()))
    assert " ".join(str(t) for t in seq[3:]) in out


def test_trace_run_replays_a_terolix_folder(folders, tmp_path):
    """bin/trace_run as a user runs it, in float32: five requests of 1, 3, 65, 2 and 66 tokens in one step,
    then two steps of a token each with the shortest leaving first.  --max-tokens counts tokens, not
    pages: the five part-filled last pages must fit all the same."""
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
