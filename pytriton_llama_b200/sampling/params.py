"""Per-request sampling settings, with lite_llama's names and defaults where it has them
(cli.py:12-16, lite_llama/generate.py:88-95): ``temperature`` 0.6, ``top_p`` 0.9, ``max_gen_len``."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    temperature: float = 0.6          # 0 = greedy (lite_llama/generate_stream.py:143-150)
    top_p: float = 0.9
    max_gen_len: Optional[int] = None  # None: up to the engine's max_seq_len (generate_stream.py:198-199)
    stop_token_ids: List[int] = field(default_factory=list)
    seed: Optional[int] = None        # None: the engine's seed
    logprobs: bool = False            # also report log softmax(logits)[token] of every generated token

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if self.max_gen_len is not None and self.max_gen_len <= 0:
            raise ValueError("max_gen_len must be positive")
