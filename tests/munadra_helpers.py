"""Small Munadra configurations and random weights for the tests, written as model folders (config.json,
model.safetensors in bfloat16).  The sizes differ from layer to layer and avoid equalities that would hide
a mix-up (unrotated size = rotated size = value size, one block, top = 1, a scale of 1)."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, Sequence

import torch

import plain_munadra as P
from terolix_helpers import tokens, write_folder  # noqa: F401  (shared by the tests)

YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def _att(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, scaling=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim, "scaling": scaling}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def _rec(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def _model(vocab, width, layers, eps=1e-5, emb=1.0, logit_scale=1.0, cap=None):
    c = {"architecture": "Munadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": emb},
         "logit_scale": logit_scale, "layers": layers}
    if cap is not None:
        c["logit_softcap"] = cap
    return c


CONFIGS: Dict[str, dict] = {
    # every mechanism, in another order than attention first; a shared latent read twice; a layer without feed-forward
    "mixed": _model(97, 64, [
        dict(_rec(48, 3, 3), mlp=_moe(5, 2, 24, 1.25)),
        dict(_att(4, 16, 8, 24, 40, 0.3, 5000.0, YARN), mlp=_dense(80)),
        dict(_att(2, 24, 8, 16, 40, 0.2, 5000.0, YARN, kv_from=1), mlp=None),
        dict(_rec(96, 1, 1), mlp=_dense(40)),
        dict(_att(3, 8, 16, 8, 24, 0.4, 300.0), mlp=_moe(3, 1, 40, 2.0)),
        dict(_att(5, 8, 8, 32, 40, 0.25, 5000.0, YARN, kv_from=1), mlp=_moe(8, 3, 16, 0.75))],
        emb=1.5, logit_scale=0.2, cap=6.0),
    # sizes that are multiples of nothing: rows on no 16-byte boundary, five taps, seven experts
    "odd": _model(131, 100, [
        dict(_att(3, 10, 6, 14, 22, 0.35, 777.0, {"factor": 2.5, "original": 48, "fast": 4.0, "slow": 0.5}), mlp=_moe(7, 4, 18, 1.0)),
        dict(_rec(75, 5, 5), mlp=None),
        dict(_att(7, 6, 6, 10, 22, 0.3, 777.0, {"factor": 2.5, "original": 48, "fast": 4.0, "slow": 0.5}, kv_from=0), mlp=_dense(52))],
        eps=3e-6),
    # sizes on which the bfloat16 tensor-core products run (16-byte rows everywhere), more heads, a long latent
    "wide": _model(320, 256, [
        dict(_att(8, 64, 32, 64, 128, 0.1, 100000.0, {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 1.0}), mlp=_moe(16, 2, 128, 3.0)),
        dict(_rec(384, 4, 4), mlp=_dense(512)),
        dict(_att(16, 32, 32, 48, 128, 0.12, 100000.0, {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 1.0}, kv_from=0), mlp=_moe(4, 4, 64, 1.5))],
        eps=1e-6, emb=0.7, logit_scale=0.4, cap=20.0),
}
# one mechanism alone (a layer needs a mixer: the feed-forwards ride on a tiny recurrent one)
CONFIGS["only_latent"] = _model(61, 64, [dict(CONFIGS["mixed"]["layers"][1], mlp=None)])
CONFIGS["only_shared"] = _model(61, 64, [dict(CONFIGS["mixed"]["layers"][1], mlp=None),
                                         dict(_att(2, 24, 8, 16, 40, 0.2, 5000.0, YARN, kv_from=0), mlp=None)])
CONFIGS["only_rglru"] = _model(61, 64, [dict(_rec(48, 3, 4), mlp=None)])
CONFIGS["only_moe"] = _model(61, 64, [dict(_rec(8, 1, 2), mlp=_moe(6, 2, 24, 1.25))])
CONFIGS["only_dense"] = _model(61, 64, [dict(_rec(8, 1, 2), mlp=_dense(136))], emb=2.0, logit_scale=0.1, cap=4.0)
# attention whose scores spread over many units, so that one key that is missed or misplaced moves the logits
CONFIGS["sharp"] = _model(53, 48, [dict(_att(3, 12, 8, 12, 20, 1.5, 2000.0, {"factor": 3.0, "original": 96, "fast": 6.0, "slow": 1.0}), mlp=None),
                                   dict(_att(2, 8, 8, 20, 20, 1.2, 2000.0, {"factor": 3.0, "original": 96, "fast": 6.0, "slow": 1.0}, kv_from=0), mlp=_dense(32))])


def tensor_shapes(c: dict) -> Dict[str, tuple]:
    W = c["width"]
    s = {"embed": (c["vocab"], W), "final.norm": (W,)}
    for i, layer in enumerate(c["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        s[p + "norm1"] = (W,)
        if layer["type"] == "rglru":
            w, B, K = m["width"], m["blocks"], m["conv"]
            s.update({p + "mix.y": (w, W), p + "mix.y.b": (w,), p + "mix.x": (w, W), p + "mix.x.b": (w,), p + "mix.conv": (w, K),
                      p + "mix.conv.b": (w,), p + "mix.ra": (B, w // B, w // B), p + "mix.ra.b": (B, w // B),
                      p + "mix.ri": (B, w // B, w // B), p + "mix.ri.b": (B, w // B), p + "mix.lam": (w,), p + "mix.o": (W, w)})
        else:
            H, d, rd, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            s.update({p + "mix.q": (H * (d + rd), W), p + "mix.uk": (H * d, r), p + "mix.uv": (H * dv, r), p + "mix.sink": (H,),
                      p + "mix.g": (H, W), p + "mix.o": (W, H * dv)})
            if m.get("kv_from") is None:
                s.update({p + "mix.dkv": (r + rd, W), p + "mix.dkv.norm": (r,)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        s[p + "norm2"] = (W,)
        if mlp["kind"] == "dense":
            s.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            f = mlp["expert"]["ff"]
            s[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                s.update({f"{p}mlp.e{e}.gate": (f, W), f"{p}mlp.e{e}.up": (f, W), f"{p}mlp.e{e}.down": (W, f)})
    return s


def random_weights(c: dict, seed: int, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices N(0, gain / sqrt(fan-in)); block norms' weights around zero (the design adds
    1), the latent's norm around 1; sinks, biases and taps of order 1/2 to 1; lambda so that the decays spread
    between fast and slow; routers wide enough that the choices differ from token to token."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif name.endswith("dkv.norm"):
            t = 1.0 + 0.2 * r
        elif name.endswith(("norm1", "norm2", "final.norm")):
            t = 0.2 * r
        elif name.endswith(".conv"):
            t = 0.6 * r
        elif name.endswith(".lam"):
            t = -2.5 + 1.5 * r
        elif name.endswith(".sink"):
            t = r
        elif name.endswith(".router"):
            t = 4.0 * r / shape[1] ** 0.5
        elif name.endswith((".ra", ".ri")):
            t = r * 1.5 / shape[2] ** 0.5
        elif len(shape) == 2 and not name.endswith(".b"):
            t = r * gain / shape[1] ** 0.5
        else:
            t = 0.5 * r
        out[name] = t.to(torch.bfloat16)
    return out


def read_folder(folder: str):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    return c, {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


@functools.lru_cache(maxsize=128)
def _oracle(folder: str, toks: tuple) -> torch.Tensor:
    c, W = read_folder(folder)
    return P.forward(c, W, list(toks)).float()


def oracle_logits(folder: str, toks: Sequence[int]) -> torch.Tensor:
    """float32 logits [T, vocab] of the whole sequence from the plain implementation (computed in float64)."""
    return _oracle(folder, tuple(int(t) for t in toks))


OBSERVED: Dict[tuple, float] = {}      # (dtype, what) -> the largest row error seen, for the report at the end of a run


def assert_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str, routed_layers: int = 0) -> None:
    """Per row, the difference with its mean taken off, root mean square over the vocabulary, relative to the
    reference row's spread.  float32 (the sharp test: only the order of sums differs): 1e-4 for every row.
    bfloat16 is judged by shares, for two reasons measured on the "mixed" configuration (stream against
    the plain implementation's, layer by layer): this design norms every sublayer's result to unit size
    before it adds it, so a sublayer's rounding error enters the stream at full weight whatever the
    stream's size (the median row is off by 0.3 % after one layer and 6 % after six), and a router whose
    scores around the cut are close picks another expert than float64 does (a third of the rows in the
    last of three routed layers), which moves that row by up to its whole spread.  The same rows do so
    under every cut and batch.  Limits: half of the rows within 10 %, nine in ten within 50 %; for models of which
    three or more layers are routed (``routed_layers``; the random configurations) 25 % and 75 %."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / (ref - ref.mean(dim=-1, keepdim=True)).pow(2).mean(dim=-1).sqrt().clamp_min(1e-9)
    worst = int(err.argmax())
    key = (dtype, what.split(":")[0])
    OBSERVED[key] = max(OBSERVED.get(key, 0.0), float(err.max()))
    if dtype == "float32":
        assert float(err.max()) <= 1e-4, f"{what}: row {worst} is off by {float(err.max()):.3e} of its spread (limit 1e-04)"
        return
    half, most = float(err.quantile(0.5)), float(err.quantile(0.9))
    if err.numel() < 20:                # a handful of rows: one other choice of an expert early on colours them all
        assert half <= 3e-1, f"{what}: half of the {err.numel()} rows are off by more than {half:.3e} of their spread (limit 3e-01)"
        return
    lim_half, lim_most = (2.5e-1, 7.5e-1) if routed_layers >= 3 else (1e-1, 5e-1)
    assert half <= lim_half, f"{what}: half of the rows are off by more than {half:.3e} of their spread (limit {lim_half:.0e})"
    assert most <= lim_most, f"{what}: a tenth of the rows is off by more than {most:.3e} of their spread (limit {lim_most:.0e})"
