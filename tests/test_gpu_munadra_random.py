"""Seeded random Munadra configurations (sizes, head counts, layer order, which layers share a latent, every constant
config.json carries) through the framework against the plain implementation: a whole prompt, a prompt followed by single
tokens, and two unequal requests in one batch decoded together, in float32 and bfloat16."""
from __future__ import annotations

import random

import pytest
import torch

from munadra_helpers import assert_logits, oracle_logits, random_weights, tokens, write_folder

pytestmark = pytest.mark.gpu
N_CONFIGS = 16


def random_config(seed: int) -> dict:
    r = random.Random(seed)
    width = r.choice([48, 64, 96, 100, 160, 256, 320])
    layers, owners = [], []
    for i in range(r.randint(2, 6)):
        mlp = r.choice([None, "dense", "moe", "moe"])
        if mlp == "dense":
            mlp = {"kind": "dense", "ff": r.choice([32, 72, 128, 320, 512])}
        elif mlp == "moe":
            E = r.randint(2, 20)
            mlp = {"kind": "moe", "router": {"experts": E, "top": r.randint(1, min(E, 6))},
                   "expert": {"ff": r.choice([16, 24, 32, 64, 96, 128]), "limit": round(r.uniform(0.5, 4.0), 2)}}
        if r.random() < 0.3 and i > 0:
            blocks = r.choice([1, 2, 3, 4])
            layers.append({"type": "rglru", "mixer": {"width": blocks * r.choice([8, 16, 24, 32, 64]), "blocks": blocks, "conv": r.randint(1, 5)}, "mlp": mlp})
            continue
        heads, dim, vdim = r.randint(1, 12), r.choice([8, 16, 24, 32, 40, 64]), r.choice([8, 16, 24, 32, 48, 64])
        if owners and r.random() < 0.5:
            src = r.choice(owners)
            m = dict(layers[src]["mixer"], heads=heads, dim=dim, vdim=vdim, kv_from=src)
        else:
            rot_dim = r.choice([2, 4, 8, 16, 32, 64])
            sc = None
            if r.random() < 0.7:
                sc = {"factor": round(r.uniform(2.0, 8.0), 2), "original": r.choice([32, 64, 512, 4096]), "fast": r.choice([4.0, 8.0, 32.0]),
                      "slow": r.choice([0.5, 1.0, 2.0])}
            m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": r.choice([8, 16, 24, 32, 48, 64, 96, 128]),
                 "rot": {"base": r.choice([100.0, 10000.0, 20000.0, 500000.0]), "dims": rot_dim, "scaling": sc}}
            owners.append(i)
        m["scale"] = round(r.uniform(0.5, 2.0) / (m["dim"] + m["rot_dim"]) ** 0.5, 4)
        layers.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    c = {"architecture": "Munadra", "vocab": r.randint(50, 700), "width": width, "norm": {"eps": r.choice([1e-6, 1e-5])},
         "embedding": {"scale": r.choice([0.5, 1.0, 2.0])}, "logit_scale": r.choice([0.1, 0.25]), "layers": layers}
    if r.random() < 0.7:
        c["logit_softcap"] = r.choice([15.0, 30.0])
    return c


@pytest.mark.parametrize("seed", range(N_CONFIGS))
def test_random_configuration(seed, tmp_path_factory):
    from kuiperllama_b200.engine import Engine, SequenceInput, load_model
    c = random_config(1000 + seed)
    folder = write_folder(str(tmp_path_factory.mktemp(f"munadra-random-{seed}")), c, random_weights(c, seed))
    V = c["vocab"]
    a, b = tokens(90, V, seed=seed), tokens(37, V, seed=seed + 500)
    ref_a, ref_b = oracle_logits(folder, a), oracle_logits(folder, b)
    what = f"random {seed}"
    routed = sum(1 for l in c["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe")
    for dtype in ("float32", "bfloat16"):
        with torch.inference_mode():
            model = load_model(folder, dtype=dtype, device="cuda:0")
            eng = Engine(model, model.new_cache(max_tokens=64 * 8))
            inp = lambda slot, toks: SequenceInput(slot, list(toks), list(range(len(toks))))
            s = eng.alloc_slot()
            assert_logits(eng.step([inp(s, a)]), ref_a, dtype, f"{what}: whole", routed)
            eng.free_slot(s)
            s = eng.alloc_slot()
            rows = [eng.step([inp(s, a[:61])]).clone()] + [eng.step([inp(s, [t])]).clone() for t in a[61:]]
            assert_logits(torch.cat(rows), ref_a, dtype, f"{what}: prompt, then tokens", routed)
            eng.free_slot(s)
            s, t = eng.alloc_slot(), eng.alloc_slot()
            first = eng.step([inp(s, a[:70]), inp(t, b[:3])])
            ra, rb = [first[:70].clone()], [first[70:].clone()]
            for k in range(20):
                out = eng.step([inp(s, [a[70 + k]]), inp(t, [b[3 + k]])])
                ra.append(out[:1].clone())
                rb.append(out[1:].clone())
            eng.free_slot(s)
            for k in range(23, 37):                                       # the longer-lived request goes on alone
                rb.append(eng.step([inp(t, [b[k]])]).clone())
            eng.free_slot(t)
            assert_logits(torch.cat(ra), ref_a, dtype, f"{what}: in a batch, first request", routed)
            assert_logits(torch.cat(rb), ref_b, dtype, f"{what}: in a batch, second request", routed)
        eng.check_device_errors()
