"""The plain feed-forward: up, an activation, down."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, NormedLazy, Runtime, StepContext, register_feed_forward
from .linear import Linear, StackedInput


@register_feed_forward("dense")
class DenseFeedForward(FeedForward):
    """f = W_down act(W_up n), no bias.  ``activation``: "gelu_tanh", "silu", or "xielu", which has
    two learned numbers p, q (a tensor of two, ``names['act']``):

        z > 0:  softplus(p) z^2 + z / 2        z <= 0:  (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2

    Spec: ``hidden_size``, ``intermediate_size``, ``activation``, ``names``.  KuiperLLama's only
    feed-forward is SwiGLU (kuiper/source/model/llama3.cpp:692-718)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid, inter, n = spec["hidden_size"], spec["intermediate_size"], spec["names"]
        m = {prefix + n["up"]: TensorDecl((inter, hid)), prefix + n["down"]: TensorDecl((hid, inter))}
        if spec["activation"] == "xielu":
            m[prefix + n["act"]] = TensorDecl((2,), role="vector")
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self.hidden, self.inter = int(spec["hidden_size"]), int(spec["intermediate_size"])
        self.activation = str(spec["activation"])
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.activation!r} (known: {', '.join(sorted(ops.ACTIVATIONS))})")
        n = spec["names"]
        self.inputs = StackedInput(runtime)
        self.inputs.add("up", tensors[prefix + n["up"]])
        self.down = Linear(tensors[prefix + n["down"]], runtime)
        self.params = None
        if self.activation == "xielu":
            pq = tensors[prefix + n["act"]].to(device=runtime.device, dtype=torch.float32)
            sp = torch.nn.functional.softplus(pq)
            self.params = torch.stack([sp[0], sp[1] + 0.5]).contiguous()      # the two slopes, made once

    def forward(self, x, step: StepContext):
        if isinstance(x, NormedLazy):
            x = x.dense()
        self.inputs.forward(x)
        act = torch.empty((x.shape[0], self.inter), dtype=self.runtime.dtype, device=x.device)
        ops.activation(self.inputs.view("up"), act, self.activation, self.params)
        return self.down.forward(act, allow_partials=True)
