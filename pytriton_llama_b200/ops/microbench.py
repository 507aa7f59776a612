"""Micro-benchmarks of the hot kernels at Llama-3.2-1B shapes, one case per call:

    python -m pytriton_llama_b200.ops.microbench <case> [--reps N]

Cases: ``decode_attention`` (32 requests x 4,096 cached tokens, 268 MB of keys and values),
``decode_step_attention`` (8 requests x 4,096 tokens with rotary encoding and cache write folded in),
``gemm_decode`` (8 tokens x a [65536, 2048] weight, 268 MB), ``gemm_small`` (8 tokens x a [3072, 2048] weight: the
product for few tokens and small weights), ``gemm_prefill`` (2,048 tokens x the
gate/up weight [16384, 2048] with the SiLU*up epilogue), ``prefill_attention`` (one 2,048-token
prompt, 32 query heads of size 64; ``prefill_attention_d128``: of size 128).  ``decode_timeline`` prints, for the kernels of the middle layer of a captured decode step (a
4-layer model of the same widths, ``--batch`` requests x 4,096 cached tokens), when the first and
the last block of each grid entered, got past the wait on its predecessor, had its first operands,
finished its loop, had its results complete and left -- %globaltimer stamps, in microseconds from
the layer's first stamp: what a sum of kernel times cannot show, the gaps between dependent kernels.
``product_shapes`` times the many-token products of the model beside the library's (torch.mm).
``sampling`` times the token choice from ``--batch`` rows of 128,256 logits, greedy and with temperature and top_p.
``decode_contexts`` times one layer's decode attention at batch 1 to 16 over contexts of 4,096 to
131,072 tokens, with the split count the operator set chooses and with the cluster form alone.
Inputs are larger than the 126 MB L2 where the kernel is a stream, so
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


LLAMA_1B_WIDTHS = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
TIMELINE_KINDS = {1: "decode attention", 10: "product -> bf16", 11: "product -> float32", 12: "product + residual", 13: "product, SiLU*up",
                  20: "small product -> bf16", 21: "small product -> f32", 22: "small product + res."}
TIMELINE_STAMPS = ["entered", "wait over", "first operands", "loop done", "results complete", "done"]


def decode_timeline(batch: int, layers: int = 4, context: int = 4096) -> dict:
    """%globaltimer stamps of one captured decode step's kernels (see the module's text)."""
    import ctypes
    from ..config.engine import EngineConfig
    from ..engine.engine import Engine, StepEntry
    cfg = dict(LLAMA_1B_WIDTHS, num_hidden_layers=layers)
    pages = batch * (context // 16 + 1) + 8
    eng = Engine(None, EngineConfig(dtype="bfloat16", page_size=16, max_gpu_num_blocks=pages, max_seq_len=context + 16,
                                    max_num_seqs=max(batch, 1), max_batched_tokens=2048, compiled_model=True),
                 model_config=cfg, random_seed=0)
    gen = torch.Generator().manual_seed(0)
    reqs = [f"r{i}" for i in range(batch)]
    for r in reqs:
        done = 0
        while done < context - 8:
            n = min(2048, context - 8 - done)
            eng.step([StepEntry(r, torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist(), [])])
            done += n
    lib = eng.ops.lib
    lib.ptl_timeline_begin.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.ptl_timeline_end.restype = ctypes.c_int
    slots = 3 * (5 * layers + 4)                       # capturing a step runs it three times; the third run is the graph's
    buf = torch.zeros((slots, 16), dtype=torch.int64, device=eng.device)
    step = lambda: eng.step([StepEntry(r, [1], [0]) for r in reqs], own_logits=False)
    lib.ptl_timeline_begin(buf.data_ptr(), slots)
    step()                                              # the first step of this batch size is captured: its kernels keep their slots
    used = lib.ptl_timeline_end()
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    eng.check_device_status()
    rows = buf[:used].cpu().tolist()
    # the graph's own launches are the last third; of those the middle layer: five kernels from a q|k|v product (bf16 store) on
    per_layer = 5
    per_run = used // 3
    first = next(i for i in range(used - per_run + per_run // 2 - per_layer, used) if rows[i][0] in (10, 20))
    chosen = rows[first:first + per_layer + 1]          # ... and the next layer's first kernel, to see the hand-over
    t0 = min(v for r in chosen for v in r[1:15] if v)
    table = []
    for r in chosen:
        first_block = [round((v - t0) / 1e3, 2) if v else None for v in r[1:7]]
        last_block = [round((v - t0) / 1e3, 2) if v else None for v in r[8:14]]
        table.append({"kernel": TIMELINE_KINDS.get(r[0], str(r[0])), "first block": first_block, "last block": last_block})
    return {"case": "decode_timeline", "batch": batch, "context": context, "stamps": TIMELINE_STAMPS, "unit": "us", "kernels": table}


def product_shapes(reps: int) -> dict:
    """The many-token products of the Llama-3.2-1B shape, this library's tcgen05 kernel beside the
    library product (cuBLAS through torch.mm) on the same inputs: q|k|v, output projection, gate/up
    and down projection at 128 to 2,048 tokens.  ``ours`` includes the fused epilogue where the
    engine would use one (add into the float32 residual; SiLU*up); ``library`` is the plain
    bfloat16 product, to which the engine then adds what the epilogue would have done (``extra``:
    the SiLU*up kernel; reading the product once more in the norm that adds it to the residual)."""
    dev = torch.device("cuda:0")
    ops = CudaOps(dev)
    H, I, QKV = 2048, 8192, 3072
    rows = []
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=dev)       # larger than L2: written between timed calls

    def timed(fn):
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(reps):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            total += start.elapsed_time(end)
        return total / reps * 1e3

    for M in (128, 256, 512, 1024, 2048):
        for name, N, K, epi in (("q|k|v", QKV, H, ops.EPI_BF16), ("output", H, H, ops.EPI_ADD_F32),
                                ("gate/up", 2 * I, H, ops.EPI_SILU_MUL), ("down", H, I, ops.EPI_ADD_F32)):
            x = torch.randn(M, K, device=dev).bfloat16()
            w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
            res = torch.zeros(M, N if epi != ops.EPI_SILU_MUL else N // 2, dtype=torch.float32, device=dev)
            ours = timed(lambda: ops.gemm_tc(x, w, epi, out=res if epi == ops.EPI_ADD_F32 else None))
            lib = timed(lambda: torch.mm(x, w.t()))
            extra = 0.0
            if epi == ops.EPI_SILU_MUL:
                gu = torch.mm(x, w.t())
                extra = timed(lambda: ops.silu_mul(gu))
            elif epi == ops.EPI_ADD_F32:
                prod = torch.mm(x, w.t())
                nw = torch.ones(N, dtype=torch.float32, device=dev)
                extra = timed(lambda: ops.add_rmsnorm(prod, res, nw, 1e-5)) - timed(lambda: ops.add_rmsnorm(None, res, nw, 1e-5, dtype=torch.bfloat16))
            rows.append({"product": name, "tokens": M, "N": N, "K": K, "ours_us": round(ours, 1), "library_us": round(lib, 1),
                         "extra_us": round(extra, 1), "routed_to": "library" if ops.library_product(M, N, K, epi) else "ours"})
    ops.check_status()
    return {"case": "product_shapes", "rows": rows}


def decode_contexts(reps: int) -> dict:
    """Decode attention of one layer (rotary encoding and cache write folded in) from a captured graph,
    over batch sizes and context lengths: the split count the operator set chooses beside the
    cluster form alone (at most eight splits of a token's keys, two blocks per SM).  Each timed
    replay walks enough separate caches that none is still in L2 when its turn comes again."""
    dev = torch.device("cuda:0")
    ops = CudaOps(dev)
    nq, nkv, d, page = 32, 8, 64, 16
    inv = (1.0 / (500000.0 ** (torch.arange(0, d, 2, device=dev).float() / d))).contiguous()

    def timed(batch, ctx, splits):
        per = ctx // page
        layer_bytes = batch * per * 2 * nkv * page * d * 2
        copies = max(2, min(64, int(400e6 // layer_bytes) + 1))
        caches = [torch.randn(batch * per, 2, nkv, page, d, device=dev).bfloat16() for _ in range(copies)]
        table = torch.arange(batch * per, dtype=torch.int32, device=dev).view(batch, per)
        rows = torch.arange(batch, dtype=torch.int32, device=dev)
        pos = torch.full((batch,), ctx - 1, dtype=torch.int32, device=dev)
        slots = (rows * per * page + ctx - 1).int()
        qkv = torch.randn(batch, (nq + 2 * nkv) * d, device=dev).bfloat16()
        hints = ops.hints_for([1] * batch, [ctx] * batch)
        if splits:
            hints.decode_splits = splits

        def walk():
            for c in caches:
                ops.rope_attention(qkv, pos, inv, d, slots, c, table, rows, nq, nkv, d, page, d ** -0.5, hints=hints)
        walk()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            walk()
        sec = _time(graph.replay, reps, ops) / copies
        return round(sec * 1e6, 1), round(layer_bytes / sec / 1e9)

    table = []
    for batch in (1, 4, 8, 16):
        for ctx in (4096, 16384, 65536, 131072):
            if batch * ctx > 8 * 131072:
                continue
            pairs = batch * nkv
            cluster_form = max(1, min(296 // pairs, 8, ctx // 128))
            us, gbs = timed(batch, ctx, 0)
            us_c, gbs_c = timed(batch, ctx, cluster_form)
            table.append({"batch": batch, "context": ctx, "us": us, "GB/s": gbs, "cluster_form_splits": cluster_form,
                          "cluster_form_us": us_c, "cluster_form_GB/s": gbs_c})
    return {"case": "decode_contexts", "rows": table}


def sampling(reps: int, rows: int) -> dict:
    """Token choice from ``rows`` rows of 128,256 float32 logits: greedy, and temperature 0.6 with
    top_p 0.9 (lite_llama's defaults, cli.py:11-20), ten calls per replay of a captured graph."""
    dev = torch.device("cuda:0")
    ops = CudaOps(dev)
    vocab = 128256
    logits = (3.0 * torch.randn(rows, vocab, device=dev)).float()
    t = torch.full((rows,), 0.6, device=dev)
    p = torch.full((rows,), 0.9, device=dev)
    u = torch.rand(rows, device=dev)
    out = {"case": "sampling", "rows": rows, "vocab": vocab}
    for name, fn in (("greedy_us", lambda: ops.sample(logits, None, None, None)), ("top_p_us", lambda: ops.sample(logits, t, p, u))):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(10):
                fn()
        out[name] = round(_time(graph.replay, reps, ops) / 10 * 1e6, 1)
    return out


def run(case: str, reps: int, batch: int = 8) -> dict:
    if case == "sampling":
        return sampling(reps, batch)
    if case == "decode_timeline":
        return decode_timeline(batch)
    if case == "decode_contexts":
        return decode_contexts(reps)
    if case == "product_shapes":
        return product_shapes(reps)
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
    if case == "gemm_small":
        # the q|k|v projection of a decode step at batch 8: 8 tokens x a [3072, 2048] weight, a fresh copy
        # of the weight every call (32 copies, 403 MB) so that it comes from memory, not from L2
        m, n, k, copies = 8, 3072, 2048, 32
        x = torch.randn(m, k, device=dev).bfloat16()
        ws = [torch.randn(n, k, device=dev).bfloat16() for _ in range(copies)]
        turn = [0]

        def call():
            turn[0] += 1
            return ops.gemm_tc(x, ws[turn[0] % copies], ops.EPI_BF16)
        sec = _time(call, max(reps, copies), ops)
        return {"case": case, "us": sec * 1e6, "bytes": n * k * 2, "GB/s": n * k * 2 / sec / 1e9,
                "note": "eager launches: the time includes what the host needs per launch"}
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
    ap.add_argument("case", choices=["decode_attention", "decode_step_attention", "gemm_decode", "gemm_small", "gemm_prefill", "prefill_attention",
                                     "prefill_attention_d128", "decode_timeline", "product_shapes", "decode_contexts", "sampling"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--batch", type=int, default=8, help="decode_timeline: requests in the step; sampling: rows of logits")
    args = ap.parse_args()
    out = run(args.case, args.reps, args.batch)
    if args.case == "decode_timeline":
        print(f"decode step, batch {out['batch']}, context {out['context']}: microseconds from the layer's first stamp")
        print(f"{'kernel':24s} {'block':6s} " + " ".join(f"{s:>16s}" for s in out["stamps"]))
        for k in out["kernels"]:
            for which in ("first block", "last block"):
                print(f"{k['kernel']:24s} {which.split()[0]:6s} " + " ".join(f"{'-' if v is None else v:>16}" for v in k[which]))
    elif args.case == "decode_contexts":
        print(f"{'batch':>5s} {'context':>8s} {'us':>8s} {'GB/s':>6s}   cluster form alone: {'splits':>6s} {'us':>8s} {'GB/s':>6s}")
        for r in out["rows"]:
            print(f"{r['batch']:5d} {r['context']:8d} {r['us']:8.1f} {r['GB/s']:6d}   {'':19s} {r['cluster_form_splits']:6d} "
                  f"{r['cluster_form_us']:8.1f} {r['cluster_form_GB/s']:6d}")
    elif args.case == "product_shapes":
        print(f"{'product':8s} {'tokens':>6s} {'N':>6s} {'K':>6s} {'ours us':>9s} {'library us':>11s} {'+extra us':>10s}  routed to")
        for r in out["rows"]:
            print(f"{r['product']:8s} {r['tokens']:6d} {r['N']:6d} {r['K']:6d} {r['ours_us']:9.1f} {r['library_us']:11.1f} {r['extra_us']:10.1f}  {r['routed_to']}")
    else:
        print(json.dumps(out))


if __name__ == "__main__":
    main()
