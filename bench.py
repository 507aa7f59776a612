"""Decode and prefill throughput of the engine on one B200, Llama-3.2-1B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 and context 4096, timed on
the device with CUDA events around exactly K decode steps (a step = the engine's step function for
one token per request, plus the sampling kernel).  ``e2e`` is the same through the Python entry
point (scheduler, step, sampling, token ids back on the host every step).  ``prefill`` times one
step of 2,048 prompt tokens; ``roofline`` relates the decode step to the bytes it has to read;
``points`` holds decode at batch 1 and 64.  Peaks come from MEASURED_PEAKS.json beside this file
when it exists, else from the fallback constants below.

lite_llama times whole completions with the wall clock (examples/benchmark.py:42-74: one warm-up
completion, then ``time.time()`` around ``text_completion``; :175-190 throughput = output tokens /
seconds); ``--impl reference`` drives its ``GenerateText.generate`` on the same shape instead and
takes a decode step's time as the difference of two calls (baseline/reference_arm.py).
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MODEL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
CONTEXT = 4096
PREFILL_TOKENS = 2048


def _llama(layers, hidden, heads, kv_heads, head_dim, inter, factor, tied):
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers, "hidden_size": hidden,
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter,
            "vocab_size": 128256, "rope_theta": 500000.0,
            "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192},
            "rms_norm_eps": 1e-5, "tie_word_embeddings": tied, "max_position_embeddings": 131072}


# The default run is the Llama-3.2-1B shape (the headline configuration).  ``--shape`` runs the same
# measurements on the two larger Llama shapes with their own workloads: 3b also times a serving run
# (32 requests, prompts of 128 to 2,048 tokens, 256 generated tokens each, continuous batching);
# 1b-long decodes at the model's longest context (4 and 1 requests of 131,072 tokens).
SHAPES = {
    "1b": {"name": "Llama-3.2-1B", "model": MODEL, "context": 4096, "batch": 8, "points": "1,64", "serving": None},
    "1b-long": {"name": "Llama-3.2-1B", "model": MODEL, "context": 131072, "batch": 4, "points": "1", "serving": None},
    "3b": {"name": "Llama-3.2-3B", "model": _llama(28, 3072, 24, 8, 128, 8192, 32.0, True), "context": 2304, "batch": 32,
           "points": "1", "serving": {"requests": 32, "prompt_lo": 128, "prompt_hi": 2048, "generated": 256}},
    "8b": {"name": "Llama-3.1-8B", "model": _llama(32, 4096, 32, 8, 128, 14336, 8.0, False), "context": 8192, "batch": 64,
           "points": "1", "serving": None},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            d = json.loads(path.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"])}, "measured"
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.proc.wait()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(int(float(r[0])))
                mx.append(int(float(r[1])))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": int(statistics.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def model_bytes_and_flops(cfg, layers, elem=2):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * d * H + H * nq * d + 3 * I * H
    matmul_params = layers * per_layer            # the LM head is counted per wanted row
    weight_bytes = elem * (matmul_params + V * H) + 4 * (2 * layers + 1) * H       # elem: bytes of a weight and of a cached value
    kv_bytes_per_token = layers * 2 * nkv * d * elem
    return matmul_params, V * H, weight_bytes, kv_bytes_per_token


def reference_arm(args) -> int:
    """``--impl reference``: lite_llama's own stock generate loop on the same shape (baseline/reference_arm.py;
    nothing of this repository's engine is imported on this path).  Prints the same JSON line with
    ``"impl": "reference"``, or an ``unavailable`` line that quotes what stopped it."""
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        import reference_arm as ref
        points = [int(p) for p in args.points.split(",") if p]
        out = ref.run(MODEL, CONTEXT, PREFILL_TOKENS, args.batch, args.steps, args.warmup, points, clock_sampler=ClockSampler())
    except BaseException as e:      # whatever stops the reference is the message; this arm never fails the bench
        if isinstance(e, KeyboardInterrupt):
            raise
        reason = f"{type(e).__name__}: {e}".replace("\n", " ")[:600]
        print(json.dumps({"impl": "reference", "unavailable": reason}))
        return 0
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the true 32-bit path (CUDA-core products, compensated sums), for its own numbers")
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="which Llama shape (default: the headline 1B configuration)")
    ap.add_argument("--batch", type=int, default=None, help="decode batch (default: 8; 32 for 3b; 64 for 8b)")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    ap.add_argument("--points", default=None, help="extra decode batch sizes, comma separated ('' for none)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill measurement (profiling runs)")
    ap.add_argument("--only-prefill", action="store_true", help="measure the prefill only and print its numbers (profiling runs)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    shape = SHAPES[args.shape]
    args.batch = args.batch or shape["batch"]
    args.points = shape["points"] if args.points is None else args.points
    args.layers = args.layers or shape["model"]["num_hidden_layers"]
    if args.impl == "reference":
        if args.shape != "1b":
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm runs the headline 1B configuration only"}))
            return 0
        return reference_arm(args)
    MODEL, CONTEXT = shape["model"], shape["context"]

    import torch
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.engine import Engine, StepEntry
    from pytriton_llama_b200.engine.llm import LLM
    from pytriton_llama_b200.sampling import SamplingParams

    W, K, B = max(3, args.warmup), args.steps, args.batch
    peaks, peak_kind = load_peaks()
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    points = [int(p) for p in args.points.split(",") if p]
    max_batch = max([B] + points)
    max_seq = CONTEXT + 8
    pages = max_batch * (-(-max_seq // 16)) + 64
    ecfg = EngineConfig(dtype=args.dtype, page_size=16, max_gpu_num_blocks=pages, max_seq_len=max_seq,
                        max_num_seqs=max_batch, max_batched_tokens=PREFILL_TOKENS, compiled_model=not args.no_graph, seed=0)
    llm = LLM(None, ecfg, model_config=cfg, random_seed=0)
    engine = llm.engine
    ops = engine.ops
    dev = engine.device
    gen = torch.Generator().manual_seed(0)

    def tokens(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()

    def fill(request, n):
        """Brings a request to n cached tokens through the step function, 2,048 tokens a step."""
        done = 0
        while done < n:
            k = min(PREFILL_TOKENS, n - done)
            engine.step([StepEntry(request, tokens(k), [])])
            done += k

    def event_time(fn, reps):
        torch.cuda.synchronize(dev)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize(dev)
        return start.elapsed_time(end) / reps

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    prompt = tokens(PREFILL_TOKENS)
    times = []
    for i in range(0 if args.no_prefill else 3 + 5):
        ms = event_time(lambda: engine.step([StepEntry("prefill", prompt, [PREFILL_TOKENS - 1])]), 1)
        engine.finish("prefill")
        if i >= 3:
            times.append(ms)
    prefill_ms = statistics.median(times) if times else float("nan")
    fp32 = args.dtype == "float32"
    matmul_params, head_params, weight_bytes, kv_per_token = model_bytes_and_flops(cfg, args.layers, 4 if fp32 else 2)
    if fp32:
        # the true 32-bit path runs on the CUDA cores: its peak is FMA lanes x 2 x the clock
        props = torch.cuda.get_device_properties(dev)
        peaks["bf16_tflops"] = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
        peak_kind += "; float32 flops against 128 FMA lanes per SM at 1,965 MHz"
    nq, d = cfg["num_attention_heads"], cfg["head_dim"]
    attn_flops = args.layers * 4 * nq * d * (PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2)
    prefill_flops = 2 * matmul_params * PREFILL_TOKENS + attn_flops + 2 * head_params
    prefill = {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}

    if args.no_prefill:
        prefill = None
    if args.only_prefill:
        print(json.dumps({"prefill": prefill}))
        return 0

    # ------------------------------------------------------------------ decode, device-timed
    def decode_run(batch, steps, warmup, sample_clocks=False):
        ctx0 = CONTEXT - steps - warmup
        reqs = [f"d{batch}-{i}" for i in range(batch)]
        for r in reqs:
            fill(r, ctx0)
        feed = [[t] for t in tokens(batch)]

        def one():
            out = engine.step([StepEntry(r, f, [0]) for r, f in zip(reqs, feed)], own_logits=False)   # sampled from at once
            ops.sample(out.logits, None, None, None)
        for _ in range(warmup):
            one()
        launches0 = ops.launches
        if sample_clocks:
            with ClockSampler() as cs:
                ms = event_time(one, steps)
            clocks = cs.summary()
        else:
            ms, clocks = event_time(one, steps), None
        launches = ops.launches - launches0
        for r in reqs:
            engine.finish(r)
        return ms, launches, clocks

    ms_step, launches, clocks = decode_run(B, K, W, sample_clocks=True)
    value = B / ms_step * 1e3
    step_bytes = weight_bytes + B * (CONTEXT - K // 2) * kv_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peak_kind}

    # ------------------------------------------------------------------ decode through the Python entry point
    e2e = None
    if not args.no_e2e:
        # Prompts are cut into 2,048-token portions, so requests reach decoding a few steps apart;
        # they are sized so that none ends (and the batch never shrinks) inside the timed steps.
        ctx0 = CONTEXT - K - W - B * (-(-CONTEXT // PREFILL_TOKENS) + 1)
        params = SamplingParams(temperature=0.0, max_gen_len=None, stop_token_ids=[])
        reqs = [llm.add_request(tokens(ctx0), params) for _ in range(B)]
        # ``LLM.run`` is the loop behind ``generate``: it yields every step's tokens as host
        # integers; each step's integers (tokens, positions, block tables) go up from pinned memory
        steps = llm.run()
        while any(r.computed < len(r.prompt) for r in reqs):
            next(steps)
        for _ in range(W - 1):
            next(steps)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        produced = 0
        for _ in range(K):
            sampled, _ = next(steps)
            produced += len(sampled)
        torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t0
        graph = engine._graphs.get(B) or next(iter(engine._graphs.values()), None)
        h2d = 4 * graph.layout.size if graph else 4 * (8 * B + B * (-(-CONTEXT // 16)))
        e2e = {"value": round(produced / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
               "d2h_bytes_per_step": 4 * B, "ms_per_step": round(dt / K * 1e3, 4)}
        for r in reqs:                      # stop them: the measurement is over
            r.params.max_gen_len = len(r.output) + 1
        for _ in steps:
            pass

    pts = {}
    for pb in points:
        steps = max(16, K // 2)
        ms, _, _ = decode_run(pb, steps, W)
        pts[f"decode_b{pb}"] = round(pb / ms * 1e3, 1)

    serving = None
    if shape["serving"] and not args.no_e2e:
        # continuous batching through the Python entry point: every request's prompt in portions beside the others' decoding
        sv = shape["serving"]
        lens = torch.randint(sv["prompt_lo"], sv["prompt_hi"] + 1, (sv["requests"],), generator=gen).tolist()
        prompts = [tokens(n) for n in lens]
        params = SamplingParams(temperature=0.0, max_gen_len=sv["generated"], stop_token_ids=[])
        llm.generate(prompts, params)     # warm-up: the same workload once (as the batch shrinks, every smaller decode step is captured on first use)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        outs = llm.generate(prompts, params)
        torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t0
        made = sum(len(o) for o in outs)
        serving = {"requests": sv["requests"], "prompt_tokens": sum(lens), "generated_tokens": made, "seconds": round(dt, 3),
                   "generated_tokens_per_s": round(made / dt, 1), "all_tokens_per_s": round((made + sum(lens)) / dt, 1)}

    sc = cfg["rope_scaling"]
    out = {
        "metric": "decode_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32" if fp32 else "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": f"{shape['name']} shape, random weights (seed 0)", "layers": args.layers, "layers_of_model": MODEL["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "heads": nq, "kv_heads": cfg["num_key_value_heads"], "head_dim": d,
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"],
            "rope_scaling": f"llama3 factor {sc['factor']:g} low {sc['low_freq_factor']:g} high {sc['high_freq_factor']:g} original {sc['original_max_position_embeddings']}",
            "rms_norm_eps": cfg["rms_norm_eps"], "tie_word_embeddings": cfg["tie_word_embeddings"], "global_batch": B, "seq_len": CONTEXT,
            "page_size": 16, "parallelism": "single-gpu", "cuda_graph": not args.no_graph,
            "l2": f"inputs larger than L2: every step reads all weights ({weight_bytes / 1e9:.1f} GB) and the live cache",
        },
        "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "prefill": prefill, "roofline": roofline, "points": pts,
    }
    if serving:
        out["serving"] = serving
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
