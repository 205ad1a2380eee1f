"""A gate on a sublayer's result, computed from the sublayer's input."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorDecl
from .base import Part, ResidualGate, Runtime, register_gate
from .linear import Linear


@register_gate("sigmoid_linear")
class SigmoidLinearGate(ResidualGate):
    """result * sigmoid(R h + r), element by element: R is [hidden, hidden], r a bias (or absent).
    This part only makes R h; the sigmoid, the bias and the product happen in the norm kernel that
    takes the result into the stream.  Where the gated sublayer keeps its input projections in a
    ``StackedInput`` (attribute ``inputs``), R rides on that product; else it is a product of its
    own.  Spec: ``hidden_size``, the matrix's ``name`` and the bias's ``bias`` (None: none)."""

    @classmethod
    def manifest(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorDecl]:
        hid = spec["hidden_size"]
        m = {prefix + spec["name"]: TensorDecl((hid, hid))}
        if spec.get("bias"):
            m[prefix + spec["bias"]] = TensorDecl((hid,), role="vector")
        return m

    def __init__(self, spec, prefix, tensors, runtime: Runtime):
        super().__init__(spec, prefix, tensors, runtime)
        self._weight = tensors[prefix + spec["name"]]
        self._name = "gate:" + prefix + spec["name"]
        self.bias = None
        if spec.get("bias"):
            self.bias = tensors[prefix + spec["bias"]].to(device=runtime.device, dtype=torch.float32).contiguous()
        self._rides_on = None
        self._own: Optional[Linear] = None

    def attach(self, part: Part) -> None:
        inputs = getattr(part, "inputs", None)
        if inputs is not None and hasattr(inputs, "add"):
            inputs.add(self._name, self._weight)
            self._rides_on = inputs
        else:
            self._own = Linear(self._weight, self.runtime)
        self._weight = None

    def pre_activation(self, h: torch.Tensor) -> torch.Tensor:
        if self._rides_on is not None:
            return self._rides_on.view(self._name)
        if self._own is None:
            raise RuntimeError("the gate was not attached to the sublayer it gates")
        return self._own.forward(h)
