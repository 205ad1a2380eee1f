"""A plain, slow implementation of the Munadra decoder: whole sequences, no cache, float64 on the
CPU, one function per mechanism.  It shares no code with the package and is what the tests of
the package's Munadra parts compare against.

A model is an embedding table E (times a constant; E is also the classifier), layers and a final
norm.  A layer adds its sublayers' *normed results*:  x += N1(mixer(x));  x += N2(ff(x)), the
sublayers reading x itself, N(y) = y / sqrt(mean(y^2) + eps) * (1 + w).  Mixers: attention over a
shared latent (``latent_attention``) and a gated linear recurrence (``rglru``); feed-forwards: a gated
dense one and a mixture of experts.  ``weights`` maps tensor names to arrays; ``cfg`` is the
config.json dictionary.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def t64(a) -> torch.Tensor:
    return torch.as_tensor(a, dtype=F)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, offset: float = 0.0) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * (offset + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]) -> Tuple[List[float], float]:
    """Frequencies of the pairs and the factor on cos and sin.  Without ``scaling``: base^(-2i/dims), 1."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling is None:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def where(turns: float) -> float:        # the (fractional) pair index whose wave turns that often in `orig` positions
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, freqs: List[float], mscale: float) -> torch.Tensor:
    """x [T, ..., dims]: elements 2i and 2i+1 of the last axis form a pair, turned by position * freqs[i]."""
    T = x.shape[0]
    ang = positions.to(F)[:, None] * t64(freqs)[None, :]                     # [T, dims/2]
    shape = [T] + [1] * (x.dim() - 2) + [len(freqs)]
    cos, sin = (torch.cos(ang) * mscale).reshape(shape), (torch.sin(ang) * mscale).reshape(shape)
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * cos - v * sin
    out[..., 1::2] = v * cos + u * sin
    return out


def latent_keys(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """The latent c [T, kv_rank] (normed) and the shared rotated key part [T, rot_dim] of a sequence."""
    r, rd = m["kv_rank"], m["rot_dim"]
    d = h @ t64(W[p + "dkv"]).T
    c = rms_norm(d[:, :r], t64(W[p + "dkv.norm"]), eps)
    f, ms = yarn_frequencies(m["rot"]["dims"], float(m["rot"]["base"]), m["rot"].get("scaling"))
    pos = torch.arange(h.shape[0])
    kr = d[:, r:].clone()
    nd = m["rot"]["dims"]
    kr[:, :nd] = rotate_interleaved(kr[:, :nd], pos, f, ms)
    return c, kr


def latent_attention_weights(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                             shared: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """The softmax weights [H, T, T] (rows sum to less than 1: the sink takes its share), the values [T, H, vdim]
    and (c, k_rot)."""
    T = h.shape[0]
    H, d, rd, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    c, kr = shared if shared is not None else latent_keys(h, W, p, m, eps)
    q = (h @ t64(W[p + "q"]).T).reshape(T, H, d + rd)
    qn, qr = q[..., :d], q[..., d:].clone()
    f, ms = yarn_frequencies(m["rot"]["dims"], float(m["rot"]["base"]), m["rot"].get("scaling"))
    nd = m["rot"]["dims"]
    qr[..., :nd] = rotate_interleaved(qr[..., :nd], torch.arange(T), f, ms)
    kn = (c @ t64(W[p + "uk"]).T).reshape(T, H, d)
    v = (c @ t64(W[p + "uv"]).T).reshape(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * float(m["scale"])
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask[None], -math.inf)
    sink = t64(W[p + "sink"])                                            # one more term in every denominator
    top = torch.maximum(s.max(dim=-1).values, sink[:, None])
    e = torch.exp(s - top[..., None])
    return e / (e.sum(dim=-1) + torch.exp(sink[:, None] - top))[..., None], v, (c, kr)


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                     shared: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """h [T, width] -> ([T, width], (c, k_rot)).  ``shared``: another layer's latent and rotated key part."""
    T = h.shape[0]
    w, v, latent = latent_attention_weights(h, W, p, m, eps, shared)
    o = torch.einsum("hij,jhd->ihd", w, v)
    o = o * torch.sigmoid(h @ t64(W[p + "g"]).T)[..., None]
    return o.reshape(T, m["heads"] * m["vdim"]) @ t64(W[p + "o"]).T, latent


def rglru(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict) -> torch.Tensor:
    T = h.shape[0]
    w, B, taps = m["width"], m["blocks"], m["conv"]
    y = gelu_tanh(h @ t64(W[p + "y"]).T + t64(W[p + "y.b"]))
    xin = h @ t64(W[p + "x"]).T + t64(W[p + "x.b"])
    cw = t64(W[p + "conv"])                                              # [w, taps], the last column is the current token's
    padded = torch.cat([torch.zeros(taps - 1, w, dtype=F), xin], dim=0)
    u = t64(W[p + "conv.b"]).expand(T, w).clone()
    for k in range(taps):
        u = u + padded[k:k + T] * cw[:, k]
    ub = u.reshape(T, B, w // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, t64(W[p + "ra"])) + t64(W[p + "ra.b"])).reshape(T, w)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, t64(W[p + "ri"])) + t64(W[p + "ri.b"])).reshape(T, w)
    log_a = -8.0 * r * torch.nn.functional.softplus(t64(W[p + "lam"]))
    a = torch.exp(log_a)
    b = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(w, dtype=F)
    out = torch.empty(T, w, dtype=F)
    for t in range(T):
        S = a[t] * S + b[t]
        out[t] = S
    return (out * y) @ t64(W[p + "o"]).T


def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = h @ t64(W[p + "gate"]).T
    return (g * torch.sigmoid(g) * (h @ t64(W[p + "up"]).T)) @ t64(W[p + "down"]).T


def expert(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ t64(W[p + "gate"]).T, max=limit)
    u = torch.clamp(h @ t64(W[p + "up"]).T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t64(W[p + "down"]).T


def route(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The chosen experts [T, top] and their weights: softmax over all experts, the largest, not renormalised."""
    s = torch.softmax(h @ t64(W[p + "router"]).T, dim=-1)
    wgt, idx = torch.topk(s, top, dim=-1)
    return idx, wgt


def moe_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    idx, wgt = route(h, W, p, mlp["router"]["top"])
    out = torch.zeros_like(h)
    for e in range(mlp["router"]["experts"]):
        rows, slot = (idx == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += wgt[rows, slot][:, None] * expert(h[rows], W, f"{p}e{e}.", float(mlp["expert"]["limit"]))
    return out


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    E = t64(W["embed"])
    x = E[torch.as_tensor(tokens, dtype=torch.long)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    latents, layers = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "latent_attention":
            y, latents[i] = latent_attention(x, W, p + "mix.", m, eps, latents.get(m.get("kv_from")) if m.get("kv_from") is not None else None)
        else:
            y = rglru(x, W, p + "mix.", m)
        x = x + rms_norm(y, t64(W[p + "norm1"]), eps, 1.0)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, W, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, W, p + "mlp.", mlp)
            x = x + rms_norm(y, t64(W[p + "norm2"]), eps, 1.0)
        layers.append(x.clone())
    z = rms_norm(x, t64(W["final.norm"]), eps, 1.0) @ E.T * float(cfg.get("logit_scale", 1.0))
    cap = cfg.get("logit_softcap")
    if cap:
        z = float(cap) * torch.tanh(z / float(cap))
    return (z, layers) if return_layers else z
