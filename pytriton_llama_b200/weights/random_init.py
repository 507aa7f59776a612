"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

lite_llama has no such mode (its layers start from torch's defaults,
lite_llama/models/llama.py:22-24); matrices here are N(0, initializer_range), norm weights 1 or
1 + N(0, 0.01).  Values are drawn on the CPU in float32 in the sorted order of the tensor names,
so that a folder depends on nothing but configuration, seed and stored element type.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Optional, Union

import torch

from ..parts.base import TensorSpec
from .safetensors_io import write_file


def random_tensors(expected: Dict[str, TensorSpec], seed: int, std: float, dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32)
        elif spec.init == "ones_jitter":
            t = 1.0 + 0.01 * torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        elif spec.init == "normal":
            t = std * torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        else:
            raise ValueError(f"tensor {name}: unknown init {spec.init!r}")
        out[name] = t.to(dtype)
    return out


def random_tensors_on_device(expected: Dict[str, TensorSpec], seed: int, std: float, dtype: torch.dtype,
                             device) -> Dict[str, torch.Tensor]:
    """The same distributions drawn with the device's generator (other numbers than the CPU draws):
    for models too large to be worth a round trip through a file, as in benchmarks."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
        elif spec.init == "ones_jitter":
            t = 1.0 + 0.01 * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
        elif spec.init == "normal":
            t = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device).mul_(std)
        else:
            raise ValueError(f"tensor {name}: unknown init {spec.init!r}")
        out[name] = t.to(dtype)
    return out


def write_random_model(folder: Union[str, Path], config: Dict, seed: int = 0,
                       dtype: torch.dtype = torch.bfloat16, norm_init: str = "ones",
                       std: Optional[float] = None) -> Path:
    """``config`` is the content of config.json (its ``architectures`` picks the model)."""
    from ..config.registry import resolve_architecture
    from ..models.decoder import DecoderModel
    from ..parts.base import Runtime

    arch = resolve_architecture(config)
    cfg = arch.config_from_dict(config)
    spec = arch.spec_from_config(cfg, norm_init=norm_init)
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32, ops=None))
    expected = model.expected_tensors()
    tensors = random_tensors(expected, seed, spec.initializer_range if std is None else std, dtype)
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    stored = dict(cfg.to_dict()) if hasattr(cfg, "to_dict") else dict(config)
    stored["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    (folder / "config.json").write_text(json.dumps(stored, indent=2))
    write_file(folder / "model.safetensors", tensors)
    return folder
