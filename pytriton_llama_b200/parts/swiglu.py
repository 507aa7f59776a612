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

    fuses_residual = True   # forward() may add its output into the residual itself and return None
    accepts_normed = True   # x may be a norm's prepared input (the gate/up product finishes the norm)
    emits_normed = True     # the down product may prepare the input of the norm that follows

    def load(self, tensors) -> None:
        ops = self.rt.ops
        self.alternating = bool(ops is not None and hasattr(ops, "fused_ffn_layout")
                                and ops.fused_ffn_layout(self.rt.dtype, self.hidden, self.inter))
        if self.alternating:
            # rows gate_0, up_0, gate_1, up_1, ...: each accumulator row/column pair of the product
            # holds a gate and its up value, so the product's epilogue can apply SiLU(gate)*up
            gu = torch.stack([tensors["gate"], tensors["up"]], dim=1).reshape(2 * self.inter, self.hidden)
        else:
            gu = torch.cat([tensors["gate"], tensors["up"]], dim=0)
        self.w_gate_up = self._to_compute(gu)
        self.w_down = self._to_compute(tensors["down"])

    def forward(self, x, residual=None, next_norm=None):
        ops = self.rt.ops
        if self.alternating:
            h = ops.gate_up_silu(x, self.w_gate_up)
        else:
            h = ops.silu_mul(ops.linear(x, self.w_gate_up))
        if residual is not None:
            if next_norm is not None and getattr(ops, "fuses_next_norm", False):
                return ops.linear_add(h, self.w_down, residual, next_norm=next_norm)
            return ops.linear_add(h, self.w_down, residual)   # None when the product's epilogue did the add
        return ops.linear(h, self.w_down)
