"""Rotary position encoding with optional llama3 frequency scaling.

lite_llama/models/RotaryEmbedding.py:51 gives inv_freq_j = theta^(-2j/d); :80-98 rescale it for
rope_type "llama3" (wavelengths above original/low_freq_factor divided by ``factor``, a smooth
blend down to original/high_freq_factor).  The angle of position p is float32(p) * inv_freq_j
(:200-217) and the pairs (x_j, x_{j+d/2}) are turned (lite_llama/kernels/rope_emb.py:94-103).
The table of frequencies is built once on the host in float32; the rotation itself happens in
the fused cache-write kernel.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .base import Part, PartSpec, Runtime, register_part


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[dict], rotary_dim: Optional[int] = None) -> torch.Tensor:
    rot = head_dim if rotary_dim is None else rotary_dim
    exponents = torch.arange(0, rot, 2, dtype=torch.int64).to(torch.float32) / rot
    inv_freq = 1.0 / (theta ** exponents)
    if scaling is None or scaling.get("rope_type", "default") == "default":
        return inv_freq
    if scaling["rope_type"] != "llama3":
        raise ValueError(f"unknown rope scaling {scaling['rope_type']!r}")
    factor = scaling["factor"]
    low = scaling["low_freq_factor"]
    high = scaling["high_freq_factor"]
    original = scaling["original_max_position_embeddings"]
    wavelen = 2 * math.pi / inv_freq
    divided = torch.where(wavelen > original / low, inv_freq / factor, inv_freq)
    blend = (original / wavelen - low) / (high - low)
    blended = (1 - blend) * divided / factor + blend * divided
    in_band = ~(wavelen < original / high) & ~(wavelen > original / low)
    return torch.where(in_band, blended, divided)


@register_part("position", "rope")
class RotaryPosition(Part):
    """params: ``head_dim``, ``theta``, ``scaling`` (None or the llama3 block), optional ``rotary_dim``."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.head_dim = int(p["head_dim"])
        self.rot = int(p.get("rotary_dim") or self.head_dim)
        if self.rot % 2 or self.rot > self.head_dim:
            raise ValueError(f"rotary width {self.rot} must be even and at most the head size {self.head_dim}")
        # layers with the same parameters share one table on the device: an operator set that works
        # out a step's angles once for all layers tells tables apart by their address
        scaling = p.get("scaling")
        key = ("rope", self.head_dim, self.rot, float(p["theta"]), tuple(sorted(scaling.items())) if scaling else None)
        shared = getattr(runtime, "_shared_tables", None)
        if shared is None:
            shared = {}
            try:
                setattr(runtime, "_shared_tables", shared)
            except AttributeError:          # (a runtime that takes no new attributes: every part keeps its own table)
                pass
        if key not in shared:
            shared[key] = rope_inverse_frequencies(self.head_dim, float(p["theta"]), scaling, self.rot).to(runtime.device)
        self.inv_freq = shared[key]

    def rotary_table(self) -> Optional[Tuple[torch.Tensor, int]]:
        return self.inv_freq, self.rot

    def apply(self, qk: torch.Tensor, positions: torch.Tensor, heads: int, head_dim: int) -> None:
        """Never called by the mixer, which hands ``rotary_table()`` to the kernels that rotate while
        they write the cache; kept for callers that want the rotation alone (in place)."""
        half = self.rot // 2
        ang = positions.to(torch.float32)[:, None] * self.inv_freq[None, :half]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x = qk.view(qk.shape[0], heads, head_dim) if qk.is_contiguous() else qk.unflatten(1, (heads, head_dim))
        x1, x2 = x[..., :half].float(), x[..., half:self.rot].float()       # (views of x when it is float32: both results first)
        y1, y2 = (x1 * cos - x2 * sin).to(qk.dtype), (x2 * cos + x1 * sin).to(qk.dtype)
        x[..., :half] = y1
        x[..., half:self.rot] = y2


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q and k go to the cache as projected."""

    def rotary_table(self):
        return None, 0

    def apply(self, qk, positions, heads, head_dim) -> None:
        pass
