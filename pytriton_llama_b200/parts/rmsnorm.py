"""RMSNorm with the residual add fused in.

lite_llama/kernels/skip_rmsnorm.py:122-156: the block's input is added to the residual first, the
sum becomes the new residual, then y = sum / sqrt(mean(sum^2) + eps) * weight (eps inside the
root, plain weight).  Here the sum and the residual are float32 in every compute type, and y is
rounded once.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import Part, PartSpec, Runtime, TensorSpec, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """params: ``width``, ``eps``; optional ``init`` ("ones" or "ones_jitter").  Tensor: ``weight`` [width]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.width,), init=self.spec.params.get("init", "ones"))}

    def load(self, tensors) -> None:
        self.weight = self._to_f32(tensors["weight"])  # norm weights stay 32-bit in every compute type

    deferrable = True   # the product before this norm may prepare its input, the product after it finish it

    def forward(self, x, residual, rows=None):
        """``x`` may be the prepared input that a product's epilogue made for this very norm (it has
        ``materialise``): the sum is in ``residual`` already, and it is handed on as it is for the
        next product to finish.  One made for another norm, or with ``rows``, only means that
        nothing is left to add."""
        if hasattr(x, "materialise"):
            if x.weight is self.weight and rows is None:
                return x, residual
            x = None
        return self.rt.ops.add_rmsnorm(x, residual, self.weight, self.eps, rows=rows, dtype=self.rt.dtype)
