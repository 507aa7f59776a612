"""A single-GPU inference engine for the dense GQA Llama decoder, written for NVIDIA B200
(sm_100a): typed configuration and registry, safetensors weights, a decoder put together from
parts, a paged cache, one step function for mixed batches, a scheduler, sampling, and
hand-written CUDA kernels loaded from ``csrc/``.
"""
from .config import EngineConfig, LlamaConfig  # noqa: F401
from .sampling import SamplingParams  # noqa: F401

__all__ = ["EngineConfig", "LlamaConfig", "SamplingParams", "LLM", "Engine", "StepEntry",
           "GenerateText", "GenerateStreamText"]


def __getattr__(name):
    if name in ("LLM", "GenerateText", "GenerateStreamText"):
        from .engine import llm
        return getattr(llm, name)
    if name in ("Engine", "StepEntry"):
        from .engine import engine
        return getattr(engine, name)
    raise AttributeError(name)
