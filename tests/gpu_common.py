"""Helpers of the GPU tests: engines over tiny models and the comparison rules."""
from __future__ import annotations

import torch

import plain_llama
from conftest import BF16_MAX_REL, BF16_MEAN_REL, FP32_TOL, PAGE_SIZE

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def stored_dtype(dtype: str):
    """Weights are stored in the engine's compute type so that both sides read the same numbers."""
    return DTYPES[dtype]


def make_engine(folder, name, dtype, pages, max_seq_len=512, max_num_seqs=4, **extra):
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.engine import Engine
    cfg = EngineConfig(dtype=dtype, page_size=PAGE_SIZE[name], max_gpu_num_blocks=pages, max_seq_len=max_seq_len,
                       max_num_seqs=max_num_seqs, **extra)
    return Engine(folder, cfg, device="cuda:0")


def reference_logits(folder, seqs):
    cfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    return {r: plain_llama.forward(cfg, w, s) for r, s in seqs.items()}


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: str, what=""):
    got = got.double().cpu()
    ref = ref.double()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert torch.isfinite(got).all(), what
    diff = (got - ref).abs()
    if dtype == "float32":
        assert diff.max() < FP32_TOL, f"{what}: max |diff| {diff.max():.3e} at {divmod(int(diff.argmax()), ref.shape[-1])}"
    else:
        scale = max(1.0, float(ref.abs().max()))
        worst = divmod(int(diff.argmax()), ref.shape[-1])
        assert diff.max() < BF16_MAX_REL * scale, f"{what}: max |diff| {diff.max():.3e} (scale {scale:.2f}) at {worst}"
        assert diff.mean() < BF16_MEAN_REL * scale, f"{what}: mean |diff| {diff.mean():.3e} (scale {scale:.2f})"
