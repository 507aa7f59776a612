"""Interfaces and registry of the parts a decoder layer is put together from.

A part is one of five categories: ``mixer`` (attention here), ``ffn``, ``norm``, ``position``
and ``block`` (how the other four are arranged around the residual stream).  A part is described
by a ``PartSpec`` (kind + its sizes and constants + where its tensors are in the checkpoint) and
built by ``build_part``; it never sees the model's configuration and does not know which model
it is in.  New kinds are added with ``register_part`` from anywhere, tests included.

Contracts (``T`` = tokens of the step, all tensors on the runtime's device):

* every part: ``tensor_specs() -> {local name: TensorSpec}``, ``load(tensors)`` with the same
  local names (tensors in the checkpoint's stored element type, on the CPU);
* norm: ``forward(x, residual, rows=None) -> (y, residual)`` -- adds ``x`` ([T, H], or None when
  the sub-layer before already added its output) into the float32 ``residual`` (None at the first
  layer), returns the normed sum in the compute type;
* position: ``rotary_table() -> (inv_freq float32 [rot/2], rot)`` when it is a rotation of the
  (j, j + rot/2) pairs of every head by position * inv_freq[j], which the kernels apply while they
  write the cache; ``(None, 0)`` for no encoding at all; ``None`` for anything else, and then the
  mixer calls ``apply(qk, positions, heads, head_dim)`` on the projected q and k before they are
  stored (in place; ``qk`` is the [T, heads*head_dim] view of the projection's q and k columns,
  whose rows are not contiguous);
* mixer: ``cache_need() -> CacheNeed``; ``forward(x, ctx, cache) -> [T, H]`` where ``ctx`` is the
  step's ``StepContext`` and ``cache`` the ``LayerCacheView`` of the cache entry this run of the
  layer uses (``cache.write`` tells whether this run stores its keys and values);
* ffn: ``forward(x) -> [T, H]``;
* a mixer or ffn with the class attribute ``fuses_residual = True`` is called with
  ``residual=<float32 [T, H]>`` as well and may add its output into it and return None;
* block: ``forward(x, residual, ctx, cache) -> (x, residual)``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional, Tuple

import torch

CATEGORIES = ("mixer", "ffn", "norm", "position", "block")


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    init: str = "normal"      # "normal": N(0, std) | "ones" | "ones_jitter": 1 + N(0, 0.01)
    optional: bool = False    # may be absent from the checkpoint (the part then gets None)


@dataclass
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)   # local name -> checkpoint name
    parts: Dict[str, "PartSpec"] = field(default_factory=dict)  # nested parts (a mixer's position encoding)


@dataclass(frozen=True)
class CacheNeed:
    """What one run of a mixer keeps between steps.

    ``kind``: "full" (every key and value), "window" (only the last ``window`` positions) or
    "none".  ``state_shape``/``state_dtype``: per-request state of fixed size (None if none)."""
    kind: str = "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: Optional[Tuple[int, ...]] = None
    state_dtype: Optional[torch.dtype] = None

    def group_key(self):
        return (self.kind, self.kv_heads, self.head_dim, self.window, self.state_shape, self.state_dtype)


@dataclass
class Runtime:
    """Where and how parts compute: device, compute element type and the operator set."""
    device: torch.device
    dtype: torch.dtype
    ops: Any


_REGISTRY: Dict[str, Dict[str, Callable[..., Any]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str):
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; known: {CATEGORIES}")

    def deco(cls):
        _REGISTRY[category][kind] = cls
        return cls
    return deco


def part_kinds(category: str):
    return sorted(_REGISTRY[category])


def build_part(category: str, spec: PartSpec, runtime: Runtime):
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        raise KeyError(f"no {category} part of kind {spec.kind!r}; registered: {part_kinds(category)}") from None
    return cls(spec, runtime)


class Part:
    """Base of all parts: keeps the spec and the runtime, has no tensors by default."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.spec = spec
        self.rt = runtime

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Dict[str, Optional[torch.Tensor]]) -> None:
        pass

    def children(self) -> Dict[str, "Part"]:
        """Nested parts by the name they have in ``spec.parts``."""
        return {}

    # helpers for subclasses
    def _to_compute(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.rt.device, dtype=self.rt.dtype).contiguous()

    def _to_f32(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.rt.device, dtype=torch.float32).contiguous()
