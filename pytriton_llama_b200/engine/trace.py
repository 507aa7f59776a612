"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and has no model code of its own: every step goes through ``Engine.step``,
the cache manager and the kernels that generation uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places (order of entries, then of ``want``) as little-endian float32 [wanted, vocab].  After every
step a line ``done <step>`` is printed and flushed.  ``end`` lists requests whose pages are given
back after the step.  ``--max-tokens`` sizes the page pool: the most tokens that live requests
hold at any time, each request's count rounded up to a multiple of 64.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

PAGE_SIZE = 16
LIVE_REQUESTS = 8


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch
    from ..config.engine import EngineConfig
    from .engine import Engine, StepEntry

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    page = args.page_size
    pages = max(1, -(-args.max_tokens // page))
    if 64 % page:   # larger or odd pages: each request may waste up to one page beyond its 64-rounding
        pages += LIVE_REQUESTS
    cfg = EngineConfig(dtype=args.dtype, page_size=page, max_gpu_num_blocks=pages,
                       max_seq_len=max(args.max_tokens, 1), max_num_seqs=LIVE_REQUESTS)
    engine = Engine(args.model, cfg, device=args.device)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step = msg["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in msg.get("entries", [])]
        result = engine.step(entries)
        if result.logits is not None and result.logits.shape[0] > 0:
            data = result.logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
            data.tofile(out_dir / f"{step}.f32")
        else:
            torch.cuda.synchronize(engine.device)
        for rid in msg.get("end", []):
            engine.finish(rid)
        print(f"done {step}", flush=True)
    engine.check_device_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
