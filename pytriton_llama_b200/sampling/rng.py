"""Uniform numbers for sampling that depend only on (seed, request number, token index).

lite_llama draws with torch.multinomial from the global generator
(lite_llama/generate.py:40), so a request's tokens depend on its batch mates.  A counter-based
generator removes that: the same request gives the same tokens however it is batched.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, request: int, index: int) -> float:
    """A float32-exact number in [0, 1): 24 bits out of a hash of the three counters."""
    h = _splitmix64(seed & _MASK)
    h = _splitmix64(h ^ (request & _MASK))
    h = _splitmix64(h ^ (index & _MASK))
    return (h >> 40) / float(1 << 24)
