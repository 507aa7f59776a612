"""Checks a checkpoint against what a model expects and hands the tensors over by name.

lite_llama loads a converted .pth with ``strict=True`` and asserts float16
(lite_llama/executor/model_executor.py:101-125); here the safetensors file is read directly by
its own tensor names and every problem is reported in one error.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.base import TensorSpec


class WeightError(ValueError):
    """Missing, unexpected or mis-shaped tensors, all listed."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[str], wrong_type: List[str]):
        self.missing, self.unexpected = missing, unexpected
        self.wrong_shape, self.wrong_type = wrong_shape, wrong_type
        lines = ["the checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if wrong_type:
            lines.append(f"  not a floating-point tensor ({len(wrong_type)}): " + ", ".join(wrong_type))
        super().__init__("\n".join(lines))


def check_tensors(expected: Dict[str, TensorSpec], found: Dict[str, torch.Tensor],
                  ignorable: List[str] = ()) -> None:
    """Raises ``WeightError`` unless ``found`` has exactly the expected tensors with their shapes.
    Names in ``ignorable`` may be present without being expected (a stored copy of a tied head)."""
    missing = [n for n, s in expected.items() if n not in found and not s.optional]
    unexpected = [n for n in found if n not in expected and n not in ignorable]
    wrong_shape, wrong_type = [], []
    for n, s in expected.items():
        if n in found:
            t = found[n]
            if tuple(t.shape) != tuple(s.shape):
                wrong_shape.append(f"{n}: file has {list(t.shape)}, model wants {list(s.shape)}")
            if not t.dtype.is_floating_point:
                wrong_type.append(f"{n} ({t.dtype})")
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(sorted(missing), sorted(unexpected), wrong_shape, wrong_type)
