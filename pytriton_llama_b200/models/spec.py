"""A decoder described as data: which parts each layer has and in which order layers run.
(lite_llama writes the same arrangement as code: ``LlamaDecoderLayer`` with its two norms, attention
and feed-forward, and ``LlamaModel`` with a ``ModuleList`` of them run in order,
lite_llama/models/llama.py:122-163,165-225.)"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..parts.base import PartSpec


@dataclass
class RunEntry:
    """One run of a layer.  ``cache`` names the cache entry it uses (entries are numbered by the
    model; two runs that name the same entry share keys and values).  ``write`` is False when the
    run only reads what another run stored in that entry."""
    layer: int
    cache: int
    write: bool = True


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: str                      # checkpoint name of the [vocab, hidden] table
    layers: List[PartSpec]              # block specs (each with nested norm/mixer/ffn specs)
    run_order: List[RunEntry]
    final_norm: PartSpec
    lm_head: Optional[str]              # checkpoint name, or None when tied to the embedding
    initializer_range: float = 0.02
    eos_token_ids: List[int] = field(default_factory=list)
    max_position_embeddings: Optional[int] = None

    def validate(self) -> None:
        n = len(self.layers)
        writers: Dict[int, int] = {}
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < n:
                raise ValueError(f"run_order[{i}] names layer {e.layer}, but there are {n} layers")
            if e.write:
                writers.setdefault(e.cache, i)
        for i, e in enumerate(self.run_order):
            if not e.write and (e.cache not in writers or writers[e.cache] > i):
                raise ValueError(f"run_order[{i}] reads cache entry {e.cache} before any run writes it")
