"""Plain, slow Terolix decoder on the CPU in float64: the oracle of the Terolix tests.

Whole sequences from position 0, no cache, no batch, one function for each mechanism, token by
token where the design is a recurrence.  It shares no code with the package under test: the
configuration is a plain dict (config.json as it is) and the weights a plain ``{name: tensor}``
dict in float64.

The design, in this file's notation.  A model is an embedding table E, a list of layers and a
final layer norm; the logits are E x.  A layer is

    h1 = LN1(x);  x = x + LN1b(sigmoid(R1 h1 + r1) * mixer(h1))
    h2 = LN2(x);  x = x + LN2b(sigmoid(R2 h2 + r2) * ff(h2))          (no second line without a feed-forward)

with LN(x) = (x - mean) / sqrt(var + eps) * w + b.  The mixer is one of a minGRU, causal softmax
attention whose values are its unrotated keys, and a gated delta rule with short convolutions; the
feed-forward is up-projection, the xIELU activation, down-projection.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

F = torch.float64


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return {k: v.to(F) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# ----------------------------------------------------------------------------- small functions

def sigmoid(x: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b over the last axis."""
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    ap = float(softplus(torch.tensor(p, dtype=F)))
    an = 0.5 + float(softplus(torch.tensor(q, dtype=F)))
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


# ----------------------------------------------------------------------------- feed-forward and gate

def dense_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    act = w[prefix + "mlp.act"]
    z = h @ w[prefix + "mlp.up"].T
    return xielu(z, float(act[0]), float(act[1])) @ w[prefix + "mlp.down"].T


def residual_gate(h: torch.Tensor, y: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """y * sigmoid(R h + r): R = ``name``, r = ``name``.b."""
    return y * sigmoid(h @ w[name].T + w[name + ".b"])


# ----------------------------------------------------------------------------- minGRU

def mingru_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """s_t = (1 - z_t) s_(t-1) + z_t c_t with z = sigmoid(Wz h + bz), u = Wx h + bx,
    c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0); out = Wo (s_t * silu(Wg h)); s starts at zero."""
    p = prefix + "mix."
    z = sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, sigmoid(u))
    gate = silu(h @ w[p + "g"].T)
    s = torch.zeros(z.shape[1], dtype=F)
    rows = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        rows.append(s * gate[t])
    return torch.stack(rows) @ w[p + "o"].T


# ----------------------------------------------------------------------------- attention

def rotary_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i / dims), i < dims / 2, then the wavelength rule of ``rot['scaling']`` (if any)."""
    dims = int(rot["dims"])
    freqs = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for f in freqs:
            wl = 2.0 * math.pi / f
            if wl < orig / high:
                out.append(f)
            elif wl > orig / low:
                out.append(f / factor)
            else:
                s = (orig / wl - low) / (high - low)
                out.append((1.0 - s) * f / factor + s * f)
        freqs = out
    return torch.tensor(freqs, dtype=F)


def rotate_half_layout(x: torch.Tensor, freqs: torch.Tensor, positions: Sequence[int]) -> torch.Tensor:
    """x: [T, heads, dim].  Dimension i < dims/2 pairs with i + dims/2; dimensions from dims on pass."""
    half = freqs.numel()
    ang = torch.tensor(list(positions), dtype=F)[:, None] * freqs[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * half:]], dim=-1)


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, m: dict) -> torch.Tensor:
    p = prefix + "mix."
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = k                                               # the values are the keys as projected
    rot = m.get("rot")
    if rot:
        fr = rotary_frequencies(rot)
        q, kr = rotate_half_layout(q, fr, range(T)), rotate_half_layout(k, fr, range(T))
    else:
        kr = k
    out = torch.zeros(T, H, d, dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh, :] @ kr[:, g, :].T) * float(m["scale"])
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf)
        out[:, hh, :] = torch.softmax(s, dim=-1) @ v[:, g, :]
    gate = sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * d) * gate) @ w[p + "o"].T


# ----------------------------------------------------------------------------- gated delta rule

def causal_short_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x: [T, C], taps: [C, K]; y_t = sum_j taps[:, K-1-j] x_(t-j), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        if j < T:
            y[j:] += taps[:, K - 1 - j] * x[:T - j]
    return y


def delta_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, m: dict, eps: float) -> torch.Tensor:
    p = prefix + "mix."
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(causal_short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)                                             # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(d, dv, dtype=F)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hh] = S.T @ q[t, g]
    o = rms_divide(o, eps) * w[p + "norm"]
    o = o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ----------------------------------------------------------------------------- the model

def mixer(kind: str, h, w, prefix, m, eps):
    if kind == "mingru":
        return mingru_mixer(h, w, prefix)
    if kind == "attention":
        return attention_mixer(h, w, prefix, m)
    if kind == "delta":
        return delta_mixer(h, w, prefix, m, eps)
    raise ValueError(kind)


def residual_streams(w: Dict[str, torch.Tensor], c: dict, tokens: Sequence[int]) -> List[torch.Tensor]:
    """The residual stream [T, width] after every layer."""
    eps = float(c["norm"]["eps"])
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)].clone()
    out = []
    for i, layer in enumerate(c["layers"]):
        pre = f"l{i}."
        ln = lambda name, t: layer_norm(t, w[pre + name], w[pre + name + ".b"], eps)
        h = ln("norm1", x)
        y = mixer(layer["type"], h, w, pre, layer["mixer"], eps)
        x = x + ln("norm1b", residual_gate(h, y, w, pre + "rg1"))
        if layer.get("mlp") is not None:
            h = ln("norm2", x)
            y = dense_feed_forward(h, w, pre)
            x = x + ln("norm2b", residual_gate(h, y, w, pre + "rg2"))
        out.append(x)
    return out


def forward_logits(w: Dict[str, torch.Tensor], c: dict, tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    x = residual_streams(w, c, tokens)[-1]
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], float(c["norm"]["eps"]))
    return x @ w["embed"].T


def attention_weights(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, m: dict) -> torch.Tensor:
    """softmax weights [H, T, T] of one attention mixer on input h (what tests use to see which key a
    query reads most)."""
    p = prefix + "mix."
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    if m.get("rot"):
        fr = rotary_frequencies(m["rot"])
        q, k = rotate_half_layout(q, fr, range(T)), rotate_half_layout(k, fr, range(T))
    out = torch.zeros(H, T, T, dtype=F)
    for hh in range(H):
        s = (q[:, hh, :] @ k[:, hh // (H // G), :].T) * float(m["scale"])
        out[hh] = torch.softmax(s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf), dim=-1)
    return out
