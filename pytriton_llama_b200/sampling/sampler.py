"""Picks next tokens from a step's logits on the device.

lite_llama/generate.py:135-137: logits / temperature -> softmax -> ``sample_top_p`` (:30-43: sort,
cumulative sum, drop tokens whose preceding mass exceeds p, renormalise, draw); argmax when
temperature is 0 (lite_llama/generate_stream.py:143-150).  The kernel applies the same rule
without a sort and draws with a uniform number supplied per row.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .params import SamplingParams
from .rng import uniform


class Sampler:
    def __init__(self, ops, device, seed: int = 0):
        self.ops = ops
        self.device = torch.device(device)
        self.seed = seed

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], request_numbers: Sequence[int],
               token_indices: Sequence[int]) -> List[int]:
        """One token per logits row.  ``request_numbers`` and ``token_indices`` feed the counter-based
        uniform numbers (the index is the count of tokens the request has generated so far)."""
        return self.sample_with_logprobs(logits, params, request_numbers, token_indices)[0]

    def sample_with_logprobs(self, logits, params, request_numbers, token_indices):
        """(tokens, logprobs): ``logprobs[i]`` is log softmax(logits[i])[tokens[i]] of the unscaled
        logits (lite_llama/generete_with_probs.py:154-165) where ``params[i].logprobs`` is set, else None."""
        if logits is None or logits.shape[0] == 0:
            return [], []
        tokens, lp = self.sample_device(logits, params, request_numbers, token_indices)
        if lp is not None:
            both = torch.stack([tokens.to(torch.float32), lp]).tolist()     # one read-back for both
            return [int(t) for t in both[0]], [v if p.logprobs else None for v, p in zip(both[1], params)]
        return tokens.tolist(), [None] * len(params)

    def sample_device(self, logits, params, request_numbers, token_indices, out=None):
        """The same without reading anything back: (int32 tokens on the device, written to ``out``
        if given; float32 log-probabilities on the device, or None if no row asks for them)."""
        rows = logits.shape[0]
        if all(p.temperature <= 0 for p in params):
            tokens = self.ops.sample(logits, None, None, None, out=out)
        else:
            host = torch.empty((3, rows), dtype=torch.float32, pin_memory=self.device.type == "cuda")
            h = host.numpy()
            for i, p in enumerate(params):
                seed = self.seed if p.seed is None else p.seed
                h[0, i], h[1, i], h[2, i] = p.temperature, p.top_p, uniform(seed, request_numbers[i], token_indices[i])
            dev = host.to(self.device, non_blocking=True)
            tokens = self.ops.sample(logits, dev[0], dev[1], dev[2], out=out)
        lp = self.ops.token_logprobs(logits, tokens) if any(p.logprobs for p in params) else None
        return tokens, lp
