"""Small Terolix configurations and random weights for the tests, written as model folders
(config.json, model.safetensors in bfloat16) with the safetensors package, not with the package
under test.  The sizes differ from layer to layer and avoid equalities that would hide a mix-up
(heads = kv heads, key size = value size, a mixer as wide as the model)."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List, Sequence

import torch

import plain_terolix as P


def _rot(dims, base=10000.0, scaling=None):
    return {"base": base, "dims": dims, "scaling": scaling}


def _ff(n):
    return {"kind": "dense", "ff": n}


SC = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}

CONFIGS: Dict[str, dict] = {
    # every mixer twice with different sizes; a layer without a feed-forward; group sizes 2 and 1
    "mixed": {"architecture": "Terolix", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "layers": [
        {"type": "mingru", "mixer": {"width": 48}, "mlp": _ff(80)},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.2, "rot": _rot(16, 5000.0, SC)}, "mlp": None},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "conv": 3}, "mlp": _ff(72)},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.11, "rot": _rot(64)}, "mlp": _ff(40)},
        {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 64, "vdim": 16, "conv": 1}, "mlp": None},
        {"type": "mingru", "mixer": {"width": 96}, "mlp": _ff(24)}]},
    # sizes that are multiples of nothing: rows that start on no 16-byte boundary, a key size of 72 (three
    # lanes' worth and a rest), five taps, three kv heads, a rotation of 20 of 48 dimensions
    "odd": {"architecture": "Terolix", "vocab": 131, "width": 100, "norm": {"eps": 3e-6}, "layers": [
        {"type": "delta", "mixer": {"heads": 6, "kv_heads": 3, "dim": 72, "vdim": 24, "conv": 5}, "mlp": _ff(52)},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 48, "vdim": 48, "scale": 0.3, "rot": _rot(20, 300.0)}, "mlp": _ff(36)},
        {"type": "mingru", "mixer": {"width": 75}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 18, "vdim": 18, "scale": 0.25, "rot": None}, "mlp": _ff(44)}]},
    # the sizes of the tensor-core kernels: head size 128 in a group of 8, key and value size 128
    "wide": {"architecture": "Terolix", "vocab": 320, "width": 256, "norm": {"eps": 1e-6}, "layers": [
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.09, "rot": _rot(64, 500000.0, SC)}, "mlp": _ff(512)},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 2}, "mlp": _ff(192)},
        {"type": "mingru", "mixer": {"width": 384}, "mlp": _ff(128)}]},
}
# query heads in groups larger than the tensor-core decode kernel's 16: 24 on one key head, head sizes 64 and 32
CONFIGS["grouped"] = {"architecture": "Terolix", "vocab": 83, "width": 96, "norm": {"eps": 1e-5}, "layers": [
    {"type": "attention", "mixer": {"heads": 24, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.15, "rot": _rot(32, 20000.0)}, "mlp": _ff(64)},
    {"type": "attention", "mixer": {"heads": 24, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2, "rot": _rot(8)}, "mlp": None}]}
# one layer of each mechanism alone (the attention of "needle" is built by the test that uses it)
for _kind, _layer in (("mingru", CONFIGS["mixed"]["layers"][0]), ("attention", CONFIGS["mixed"]["layers"][1]),
                      ("delta", CONFIGS["mixed"]["layers"][2])):
    CONFIGS["only_" + _kind] = {"architecture": "Terolix", "vocab": 61, "width": 64, "norm": {"eps": 1e-5},
                                "layers": [dict(_layer, mlp=None)]}
CONFIGS["only_ff"] = {"architecture": "Terolix", "vocab": 61, "width": 64, "norm": {"eps": 1e-5},
                      "layers": [{"type": "mingru", "mixer": {"width": 8}, "mlp": _ff(136)}]}


def tensor_shapes(c: dict) -> Dict[str, tuple]:
    W = c["width"]
    s = {"embed": (c["vocab"], W), "final.norm": (W,), "final.norm.b": (W,)}
    for i, layer in enumerate(c["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if layer["mlp"] else ()):
            s[p + n], s[p + n + ".b"] = (W,), (W,)
        for n in ("rg1",) + (("rg2",) if layer["mlp"] else ()):
            s[p + n], s[p + n + ".b"] = (W, W), (W,)
        if layer["type"] == "mingru":
            w = m["width"]
            s.update({p + "mix.z": (w, W), p + "mix.z.b": (w,), p + "mix.x": (w, W), p + "mix.x.b": (w,), p + "mix.g": (w, W), p + "mix.o": (W, w)})
        elif layer["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            s.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.g": (H * d, W), p + "mix.o": (W, H * d)})
        else:
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            s.update({p + "mix.q": (G * d, W), p + "mix.q.conv": (G * d, K), p + "mix.k": (G * d, W), p + "mix.k.conv": (G * d, K),
                      p + "mix.v": (H * dv, W), p + "mix.v.conv": (H * dv, K), p + "mix.b": (H, W), p + "mix.a": (H, W),
                      p + "mix.A_log": (H,), p + "mix.dt_bias": (H,), p + "mix.norm": (dv,), p + "mix.g": (H * dv, W), p + "mix.o": (W, H * dv)})
        if layer["mlp"]:
            f = layer["mlp"]["ff"]
            s.update({p + "mlp.up": (f, W), p + "mlp.down": (W, f), p + "mlp.act": (2,)})
    return s


def random_weights(c: dict, seed: int, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices N(0, gain / sqrt(fan-in)) so that activations keep their size from
    layer to layer; norm weights around 1; biases, taps and the per-head numbers of order 1/2."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif name.endswith(".conv"):
            t = 0.6 * r
        elif len(shape) == 2:
            t = r * gain / shape[1] ** 0.5
        elif name.endswith(("norm", "norm1", "norm2", "norm1b", "norm2b")) and not name.endswith(".b"):
            t = 1.0 + 0.2 * r
        else:
            t = 0.5 * r
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(folder: str, c: dict, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(c, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@functools.lru_cache(maxsize=128)
def _oracle(folder: str, toks: tuple) -> torch.Tensor:
    return P.forward_logits(P.read_weights(folder), P.read_config(folder), list(toks)).float()


def oracle_logits(folder: str, toks: Sequence[int]) -> torch.Tensor:
    """float32 logits [T, vocab] of the whole sequence from the plain implementation (computed in float64)."""
    return _oracle(folder, tuple(int(t) for t in toks))


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    """Per row, the difference with its mean taken off, root mean square over the vocabulary, relative
    to the reference row's spread.  float32 (the sharp test: only the order of sums differs): 1e-4 for
    every row.  bfloat16 (every layer rounds about ten tensors to 8 bits of mantissa): most rows lie
    near 2 %, but a row whose sharp attention or delta-rule state amplifies one rounding comes to 13 or
    20 % and does so whichever way the tokens are cut into steps or batched (the same figure to four
    digits), so the limit is 5 % for nine rows in ten and 30 % for every row."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / (ref - ref.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt().clamp_min(1e-9)
    tol = 1e-4 if dtype == "float32" else 3e-1
    worst = int(err.argmax())
    assert float(err.max()) <= tol, f"{what}: row {worst} is off by {float(err.max()):.3e} of its spread (limit {tol:.0e})"
    if dtype != "float32" and err.numel() >= 10:
        q = float(err.quantile(0.9))
        assert q <= 5e-2, f"{what}: a tenth of the rows is off by more than {q:.3e} of their spread (limit 5e-02)"
