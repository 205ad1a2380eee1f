"""Recurrent mixers: a state of fixed size per sequence instead of keys and values per token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache import CacheView, StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import Mixer, NormedLazy, PositionEncoding, Runtime, StepContext, register_mixer
from .linear import Linear, StackedInput


@register_mixer("mingru")
class MinGRUMixer(Mixer):
    """A gated recurrence whose gates read only the current token:

        z = sigmoid(Wz n + bz);  u = Wx n + bx;  c = u + 1/2 where u >= 0, sigmoid(u) below
        s_t = (1 - z) s_(t-1) + z c   (element by element, s starts at zero);  out = Wo (s_t * silu(Wg n))

    The state s is float32 [width] per slot.  Spec: ``hidden_size``, ``width`` and ``names`` of
    z, x, g, o and of the two biases (z_bias, x_bias; None: none).  z, x and g are one product.
    KuiperLLama has no recurrent mixer (its mixer is mha_kernel.cu:61,74-106)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, w, n = spec["hidden_size"], spec["width"], spec["names"]
        m = {prefix + n[k]: TensorDecl((w, hid)) for k in ("z", "x", "g")}
        m[prefix + n["o"]] = TensorDecl((hid, w))
        for k in ("z_bias", "x_bias"):
            if n.get(k):
                m[prefix + n[k]] = TensorDecl((w,), role="vector")
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden, self.width = int(spec["hidden_size"]), int(spec["width"])
        n = spec["names"]
        self.inputs = StackedInput(runtime)
        for k in ("z", "x", "g"):
            self.inputs.add(k, tensors[prefix + n[k]])
        self.o = Linear(tensors[prefix + n["o"]], runtime)
        f32 = lambda name: tensors[prefix + name].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.bias_z = f32(n["z_bias"]) if n.get("z_bias") else None
        self.bias_x = f32(n["x_bias"]) if n.get("x_bias") else None

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.width,), torch.float32)

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if isinstance(x, NormedLazy):
            x = x.dense()
        proj = self.inputs.forward(x)
        col = self.inputs.column
        # rows that belong to no sequence (a small step's padding) are not written by the scan: keep them defined
        make = torch.empty if step.n_tokens == step.n_seqs else torch.zeros
        mixed = make((step.n_tokens, self.width), dtype=self.runtime.dtype, device=x.device)
        ops.mingru_scan(proj, col("z"), col("x"), col("g"), self.bias_z, self.bias_x, cache.state, mixed, step, self.width)
        return self.o.forward(mixed, allow_partials=True)


@register_mixer("gated_delta")
class GatedDeltaMixer(Mixer):
    """The gated delta rule.  q = Wq n, k = Wk n (G heads of size d), v = Wv n (H heads of size dv;
    head h reads q/k head h // (H / G)); each channel of q, k, v passes a causal convolution over
    its last ``conv`` inputs and SiLU; q and k become x / sqrt(sum x^2 + unit_eps) per head, q also
    times ``q_scale``; beta = sigmoid(Wb n) and decay = exp(-exp(A_log) softplus(Wa n + dt_bias))
    per head.  Then per head, with S [d, dv] starting at zero:

        S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q

    and out = Wo (o / rms(o) * w_norm * silu(Wg n)), the RMS over each head's dv values.  The slot's
    state is float32: S as [H, d, dv], then the last conv - 1 inputs of the convolution.  All of
    q, k, v, beta, decay and g come from one product.  Spec: ``hidden_size``, ``heads``,
    ``kv_heads``, ``dim``, ``vdim``, ``conv``, ``norm_eps``, ``unit_eps``, ``q_scale`` and ``names``.
    KuiperLLama has no recurrent mixer (its mixer is mha_kernel.cu:61,74-106)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, H, G, d, dv, K, n = (spec[k] for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim", "conv", "names"))
        return {
            prefix + n["q"]: TensorDecl((G * d, hid)), prefix + n["k"]: TensorDecl((G * d, hid)),
            prefix + n["v"]: TensorDecl((H * dv, hid)), prefix + n["g"]: TensorDecl((H * dv, hid)),
            prefix + n["beta"]: TensorDecl((H, hid)), prefix + n["a"]: TensorDecl((H, hid)),
            prefix + n["o"]: TensorDecl((hid, H * dv)),
            prefix + n["q_conv"]: TensorDecl((G * d, K), role="vector"), prefix + n["k_conv"]: TensorDecl((G * d, K), role="vector"),
            prefix + n["v_conv"]: TensorDecl((H * dv, K), role="vector"),
            prefix + n["A_log"]: TensorDecl((H,), role="vector"), prefix + n["dt_bias"]: TensorDecl((H,), role="vector"),
            prefix + n["norm"]: TensorDecl((dv,), role="vector", init="one_plus_normal"),
        }

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden = int(spec["hidden_size"])
        self.H, self.G, self.d, self.dv = int(spec["heads"]), int(spec["kv_heads"]), int(spec["dim"]), int(spec["vdim"])
        self.taps = int(spec["conv"])
        if self.H % self.G:
            raise ValueError(f"{self.H} heads are not a multiple of {self.G} key heads")
        if self.d > 256:
            raise ValueError(f"key size {self.d} is not supported by the delta-rule kernel (up to 256)")
        if self.taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {self.taps}")
        self.norm_eps, self.unit_eps = float(spec["norm_eps"]), float(spec["unit_eps"])
        self.q_scale = float(spec["q_scale"])
        n = spec["names"]
        self.inputs = StackedInput(runtime)
        dev, dt = runtime.device, runtime.dtype
        # q | k | v as one piece: the convolution runs over their channels as one range
        self.inputs.add("qkv", torch.cat([tensors[prefix + n[k]].to(device=dev, dtype=dt) for k in ("q", "k", "v")], dim=0))
        for k in ("g", "beta", "a"):
            self.inputs.add(k, tensors[prefix + n[k]])
        self.o = Linear(tensors[prefix + n["o"]], runtime)
        f32 = lambda name: tensors[prefix + name].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.conv_weight = torch.cat([f32(n[k]) for k in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.A_log, self.dt_bias, self.norm_weight = f32(n["A_log"]), f32(n["dt_bias"]), f32(n["norm"])
        self.channels = 2 * self.G * self.d + self.H * self.dv
        self.conv_off = self.H * self.dv * self.d

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.conv_off + (self.taps - 1) * self.channels,), torch.float32)

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if isinstance(x, NormedLazy):
            x = x.dense()
        proj = self.inputs.forward(x)
        col = self.inputs.column
        n = step.n_tokens
        # rows that belong to no sequence (a small step's padding) are not written by the scan: keep them defined
        make = torch.empty if n == step.n_seqs else torch.zeros
        o = make((n, self.H * self.dv), dtype=torch.float32, device=x.device)
        ops.gated_delta_rule(proj, col("qkv"), col("beta"), col("a"), self.conv_weight, self.A_log, self.dt_bias, cache.state,
                             self.conv_off, o, step, self.H, self.G, self.d, self.dv, self.q_scale, self.unit_eps)
        gated = torch.empty((n, self.H * self.dv), dtype=self.runtime.dtype, device=x.device)
        ops.head_rmsnorm_gate(o, self.inputs.view("g"), self.norm_weight, gated, self.H, self.dv, self.norm_eps)
        return self.o.forward(gated, allow_partials=True)


@register_mixer("rglru")
class RGLRUMixer(Mixer):
    """The recurrent block with a real-gated linear recurrent unit (De et al., "Griffin: Mixing Gated Linear
    Recurrences with Local Attention for Efficient Language Models", 2024).  Two branches of ``width``:

        y = gelu_tanh(Wy n + by);   u = conv(Wx n + bx)    (a causal convolution per channel over ``conv`` inputs, with bias)
        per block b of width / blocks channels:  r = sigmoid(Ra[b] u_b + ra_b),  i = sigmoid(Ri[b] u_b + ri_b)
        a = exp(-decay_scale * r * softplus(lambda));   S_t = a S_(t-1) + sqrt(1 - a^2) * i * u;   out = Wo (S_t * y)

    S starts at zero and the first token takes no other path.  The slot's state is float32: S [width], then
    the convolution's last conv - 1 inputs.  u, both gates, a and S are 32-bit in every run: the gate matrices
    are held in float32 and multiplied by the grouped product's float32 instance.  Spec: ``hidden_size``,
    ``width``, ``blocks``, ``conv``, ``decay_scale`` and ``names`` (y, x, y_bias, x_bias, conv, conv_bias, ra,
    ra_bias, ri, ri_bias, lam, o).  KuiperLLama has no recurrent mixer (its mixer is mha_kernel.cu:61,74-106)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, w, B, K, n = (spec[k] for k in ("hidden_size", "width", "blocks", "conv", "names"))
        bs = w // B
        vec = lambda shape: TensorDecl(shape, role="vector")
        return {prefix + n["y"]: TensorDecl((w, hid)), prefix + n["x"]: TensorDecl((w, hid)), prefix + n["o"]: TensorDecl((hid, w)),
                prefix + n["y_bias"]: vec((w,)), prefix + n["x_bias"]: vec((w,)), prefix + n["conv"]: vec((w, K)),
                prefix + n["conv_bias"]: vec((w,)), prefix + n["ra"]: vec((B, bs, bs)), prefix + n["ra_bias"]: vec((B, bs)),
                prefix + n["ri"]: vec((B, bs, bs)), prefix + n["ri_bias"]: vec((B, bs)), prefix + n["lam"]: vec((w,))}

    def __init__(self, spec, prefix, tensors, runtime: Runtime, position: Optional[PositionEncoding] = None):
        super().__init__(spec, prefix, tensors, runtime, position)
        self.hidden, self.width, self.blocks, self.taps = (int(spec[k]) for k in ("hidden_size", "width", "blocks", "conv"))
        if self.blocks < 1 or self.width % self.blocks:
            raise ValueError(f"a width of {self.width} does not split into {self.blocks} equal blocks")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"the convolution kernel takes 1 to 16 taps, got {self.taps}")
        self.block = self.width // self.blocks
        self.decay_scale = float(spec["decay_scale"])
        n = spec["names"]
        self.inputs = StackedInput(runtime)
        self.inputs.add("y", tensors[prefix + n["y"]])
        self.inputs.add("x", tensors[prefix + n["x"]])
        self.o = Linear(tensors[prefix + n["o"]], runtime)
        f32 = lambda name: tensors[prefix + name].to(device=runtime.device, dtype=torch.float32).contiguous()
        self.y_bias, self.x_bias, self.conv_weight, self.conv_bias = f32(n["y_bias"]), f32(n["x_bias"]), f32(n["conv"]), f32(n["conv_bias"])
        # both gates of a block from one product: [blocks, 2 block, block], recurrence-gate rows then input-gate rows
        self.gate_weight = torch.cat([f32(n["ra"]), f32(n["ri"])], dim=1).contiguous()
        self.ra_bias, self.ri_bias = f32(n["ra_bias"]).reshape(-1), f32(n["ri_bias"]).reshape(-1)
        self.softplus_lambda = torch.nn.functional.softplus(f32(n["lam"])).contiguous()      # made once, in float32

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.width * self.taps,), torch.float32)

    def forward(self, x, step: StepContext, cache: CacheView) -> torch.Tensor:
        if isinstance(x, NormedLazy):
            x = x.dense()
        n, w, dev = step.n_tokens, self.width, x.device
        proj = self.inputs.forward(x)
        y_col, x_col = self.inputs.column("y"), self.inputs.column("x")
        # rows that belong to no sequence (a small step's padding) are not written by the kernels: keep them defined
        make = torch.empty if n == step.n_seqs else torch.zeros
        u = make((n, w), dtype=torch.float32, device=dev)
        ops.causal_conv(proj, x_col, self.x_bias, self.conv_weight, self.conv_bias, cache.state, step, w, u)
        gates = torch.empty((n, 2 * w), dtype=torch.float32, device=dev)
        ops.grouped_gemm(u, self.gate_weight, gates, a_group_stride=self.block, out_group_stride=2 * self.block, rows=n,
                         tile_rows=16 if n <= 16 else 64)
        ops.rglru_gate(gates, u, self.ra_bias, self.ri_bias, self.softplus_lambda, self.decay_scale, n, w, self.block)
        mixed = make((n, w), dtype=self.runtime.dtype, device=dev)
        ops.linear_scan(gates, self.block, proj, y_col, x_col, self.y_bias, self.x_bias, self.taps, cache.state, step, w, mixed)
        return self.o.forward(mixed, allow_partials=True)
