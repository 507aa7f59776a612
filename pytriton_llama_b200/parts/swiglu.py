"""Dense SwiGLU feed-forward.

lite_llama/models/llama.py:107-120: down(silu(gate(x)) * up(x)), three bias-free projections;
silu(a) = a * sigmoid(a) in float32 (lite_llama/kernels/swiglu.py:44-46,64-66).  Gate and up are
kept as one [2*inter, hidden] weight (gate rows first) so that one product feeds the activation.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("ffn", "swiglu")
class SwiGLU(Part):
    """params: ``hidden``, ``inter``.  Tensors: ``gate``, ``up`` [inter, hidden], ``down`` [hidden, inter]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec.params["hidden"])
        self.inter = int(spec.params["inter"])
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {
            "gate": TensorSpec((self.inter, self.hidden)),
            "up": TensorSpec((self.inter, self.hidden)),
            "down": TensorSpec((self.hidden, self.inter)),
        }

    def load(self, tensors) -> None:
        self.w_gate_up = self._to_compute(torch.cat([tensors["gate"], tensors["up"]], dim=0))
        self.w_down = self._to_compute(tensors["down"])

    def forward(self, x):
        ops = self.rt.ops
        return ops.linear(ops.silu_mul(ops.linear(x, self.w_gate_up)), self.w_down)
