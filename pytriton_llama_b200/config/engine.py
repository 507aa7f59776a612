"""Settings of the engine itself (not of the model): cache geometry, batch limits, precision.

lite_llama spreads these over keyword arguments of its entry points (cli.py:11-20:
``max_seq_len``, ``max_gpu_num_blocks``, ``compiled_model``); the same meanings are kept where a
name exists there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute type {name} is not supported (bfloat16 or float32)")
        return name
    try:
        return _DTYPES[str(name)]
    except KeyError:
        raise ValueError(f"compute type {name!r} is not supported (bfloat16 or float32)") from None


@dataclass
class EngineConfig:
    dtype: torch.dtype = torch.bfloat16
    page_size: int = 16
    max_gpu_num_blocks: Optional[int] = None   # pages per cache group; None: sized from free memory
    gpu_memory_fraction: float = 0.9           # lite_llama/executor/mem_manager.py:98-108 uses 0.9 too
    max_seq_len: int = 2048                    # longest request (prompt + generated)
    max_num_seqs: int = 64                     # live requests (lite_llama's max_batch_size)
    max_batched_tokens: int = 2048             # token budget of one step
    compiled_model: bool = False               # capture decode steps in CUDA graphs
    capture_mixed_steps: bool = True           # with compiled_model: also steps that hold prompt portions (padded shapes, up to 1,024 tokens)
    graph_context_buckets: Tuple[int, ...] = (4096, 16384, 65536)   # with compiled_model: decode steps are captured per class of
                                               # context length (the key splits of attention are fixed at capture)
    overlap_steps: bool = True                 # plan and launch the next step while the last one's tokens are read
    timing: bool = False                       # diagnostic: CUDA-event time of every step and of every class of kernels; steps run
                                               # uncaptured and the host waits for each (lite_llama/generete_with_probs.py:124-126,176-182 times its loop so)
    seed: int = 0

    def __post_init__(self):
        self.dtype = parse_dtype(self.dtype)
        for name in ("page_size", "max_seq_len", "max_num_seqs", "max_batched_tokens"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")
        if self.max_gpu_num_blocks is not None and self.max_gpu_num_blocks <= 0:
            raise ValueError("max_gpu_num_blocks must be positive")
        self.graph_context_buckets = tuple(sorted(int(c) for c in self.graph_context_buckets))
        if any(c <= 0 for c in self.graph_context_buckets):
            raise ValueError("graph_context_buckets must be positive")
        if not 0 < self.gpu_memory_fraction <= 1:
            raise ValueError("gpu_memory_fraction must be in (0, 1]")
