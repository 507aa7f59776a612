"""Micro-benchmarks of the hot kernels at Llama-3.2-1B shapes, one case per call:

    python -m pytriton_llama_b200.ops.microbench <case> [--reps N]

Cases: ``decode_attention`` (32 requests x 4,096 cached tokens, 268 MB of keys and values),
``decode_step_attention`` (8 requests x 4,096 tokens with rotary encoding and cache write folded in),
``gemm_decode`` (8 tokens x a [65536, 2048] weight, 268 MB), ``gemm_prefill`` (2,048 tokens x the
gate/up weight [16384, 2048] with the SiLU*up epilogue), ``prefill_attention`` (one 2,048-token
prompt, 32 query heads of size 64; ``prefill_attention_d128``: of size 128).  Inputs are larger than the 126 MB L2 where the kernel is a stream, so
DRAM figures mean something, yet small enough for a profiler to replay.  Each case prints its
time from CUDA events after warm-up and the bytes or FLOPs per second that follow from it.
lite_llama benchmarks its Triton kernels the same way from their ``__main__`` blocks
(lite_llama/kernels/flashdecoding.py:289-333).
"""
from __future__ import annotations

import argparse
import json
from types import SimpleNamespace

import torch

from .cuda import CudaOps


def _time(fn, reps: int, ops: CudaOps) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    end.record()
    torch.cuda.synchronize()
    ops.check_status()          # a kernel whose waits ran out would have been timed for nothing
    return start.elapsed_time(end) / reps * 1e-3


def run(case: str, reps: int) -> dict:
    dev = torch.device("cuda:0")
    ops = CudaOps(dev)
    nq, nkv, d, page = 32, 8, 64, 16
    if case == "decode_attention":
        batch, ctx = 32, 4096
        per = ctx // page
        cache = torch.randn(batch * per, 2, nkv, page, d, device=dev).bfloat16()
        table = torch.arange(batch * per, dtype=torch.int32, device=dev).view(batch, per)
        rows = torch.arange(batch, dtype=torch.int32, device=dev)
        pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=dev)
        qkv = torch.randn(batch, (nq + 2 * nkv) * d, device=dev).bfloat16()
        hints = ops.hints_for([1] * batch, [ctx] * batch)
        sec = _time(lambda: ops.paged_attention(qkv, cache, table, rows, pos, nq, nkv, d, page, d ** -0.5, hints=hints), reps, ops)
        return {"case": case, "us": sec * 1e6, "bytes": cache.numel() * 2, "GB/s": cache.numel() * 2 / sec / 1e9}
    if case == "decode_step_attention":
        # the attention of one layer of a decode step at batch 8: q|k|v unrotated, rotary encoding and
        # the cache write inside the kernel, the four splits of a token merged over a cluster
        batch, ctx = 8, 4096
        per = ctx // page
        cache = torch.randn(batch * per, 2, nkv, page, d, device=dev).bfloat16()
        table = torch.arange(batch * per, dtype=torch.int32, device=dev).view(batch, per)
        rows = torch.arange(batch, dtype=torch.int32, device=dev)
        pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=dev)
        slots = (rows * per * page + ctx - 1).int()
        inv = (1.0 / (500000.0 ** (torch.arange(0, d, 2, device=dev).float() / d))).contiguous()
        qkv = torch.randn(batch, (nq + 2 * nkv) * d, device=dev).bfloat16()
        hints = ops.hints_for([1] * batch, [ctx] * batch)
        sec = _time(lambda: ops.rope_attention(qkv, pos, inv, d, slots, cache, table, rows, nq, nkv, d, page, d ** -0.5,
                                               hints=hints), reps, ops)
        nbytes = cache.numel() * 2
        return {"case": case, "us": sec * 1e6, "bytes": nbytes, "GB/s": nbytes / sec / 1e9}
    if case == "gemm_decode":
        m, n, k = 8, 65536, 2048
        x = torch.randn(m, k, device=dev).bfloat16()
        w = torch.randn(n, k, device=dev).bfloat16()
        sec = _time(lambda: ops.gemm_tc(x, w, ops.EPI_BF16), reps, ops)
        return {"case": case, "us": sec * 1e6, "bytes": n * k * 2, "GB/s": n * k * 2 / sec / 1e9}
    if case == "gemm_prefill":
        m, n, k = 2048, 16384, 2048
        x = torch.randn(m, k, device=dev).bfloat16()
        w = torch.randn(n, k, device=dev).bfloat16()
        sec = _time(lambda: ops.gemm_tc(x, w, ops.EPI_SILU_MUL), reps, ops)
        return {"case": case, "us": sec * 1e6, "flops": 2 * m * n * k, "TFLOP/s": 2 * m * n * k / sec / 1e12}
    if case in ("prefill_attention", "prefill_attention_d128"):
        if case.endswith("d128"):
            d = 128
        tokens = 2048
        pages = tokens // page
        cache = torch.randn(pages, 2, nkv, page, d, device=dev).bfloat16()
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        rows = torch.zeros(tokens, dtype=torch.int32, device=dev)
        pos = torch.arange(tokens, dtype=torch.int32, device=dev)
        qkv = torch.randn(tokens, (nq + 2 * nkv) * d, device=dev).bfloat16()
        hints = ops.hints_for([tokens], [tokens])
        sec = _time(lambda: ops.paged_attention(qkv, cache, table, rows, pos, nq, nkv, d, page, d ** -0.5, hints=hints), reps, ops)
        flops = 4 * nq * d * tokens * (tokens + 1) // 2
        return {"case": case, "us": sec * 1e6, "flops": flops, "TFLOP/s": flops / sec / 1e12}
    raise SystemExit(f"unknown case {case!r}")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=["decode_attention", "decode_step_attention", "gemm_decode", "gemm_prefill", "prefill_attention",
                                     "prefill_attention_d128"])
    ap.add_argument("--reps", type=int, default=10)
    args = ap.parse_args()
    print(json.dumps(run(args.case, args.reps)))


if __name__ == "__main__":
    main()
