"""Command line in the manner of lite_llama's cli.py (cli.py:11-20,40-66): the same option names
with the same meaning (``temperature`` 0.6, ``top_p`` 0.9, ``max_seq_len`` 2048,
``max_gpu_num_blocks``, ``max_gen_len`` 1024, ``compiled_model``), a prompt loop that streams the
answer and stops at ``exit``.  lite_llama hard-codes the checkpoint folder (cli.py:8); here it is
``--checkpoints_dir``, or ``--random_weights`` with ``--config`` and ``--seed`` to make a folder of
random weights first.  Without a tokenizer in the folder, prompts are lists of token ids.  Text
prompts are wrapped in the Llama 3 chat form with the conversation so far, as lite_llama wraps its
lines in a template (cli.py:26,49-50), when the tokenizer knows the role headers (``--raw_prompt``: never).

    python cli.py --checkpoints_dir DIR --prompt_ids 1 2 3 --max_gen_len 16 --temperature 0
    python cli.py --random_weights /tmp/m --config tiny.json --seed 1     # then the prompt loop
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Generate with the B200 Llama engine")
    ap.add_argument("--checkpoints_dir", help="model folder: config.json and model.safetensors")
    ap.add_argument("--random_weights", metavar="DIR", help="write a random-weights model folder here and use it")
    ap.add_argument("--config", help="config.json for --random_weights")
    ap.add_argument("--seed", type=int, default=0, help="seed of random weights and of sampling")
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--top_p", type=float, default=0.9)
    ap.add_argument("--max_seq_len", type=int, default=2048)
    ap.add_argument("--max_gpu_num_blocks", type=int, default=None, help="cache pages; default: from free memory")
    ap.add_argument("--max_gen_len", type=int, default=1024)
    ap.add_argument("--compiled_model", action="store_true", help="run decode steps from CUDA graphs")
    ap.add_argument("--load_model", action="store_true", default=True, help="kept for lite_llama's name; always on")
    ap.add_argument("--triton_weight", action="store_true", default=True, help="kept for lite_llama's name; no effect")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--page_size", type=int, default=16)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--stats", action="store_true",
                    help="time every step on the device (steps then run uncaptured, one at a time) and print, after each "
                         "answer, steps, tokens, tokens/s, pages in use and milliseconds by class of kernels")
    ap.add_argument("--raw_prompt", action="store_true",
                    help="text prompts go to the model as they are; default: the Llama 3 chat form (with the conversation so far) "
                         "when the tokenizer knows its role headers")
    ap.add_argument("--system", default="", help="system message of the chat form")
    ap.add_argument("--prompt", help="one text prompt (needs a tokenizer in the model folder)")
    ap.add_argument("--prompt_ids", type=int, nargs="+", help="one prompt as token ids")
    return ap


def _has_tokenizer(folder: Path) -> bool:
    return any((folder / n).is_file() for n in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json"))


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    if args.random_weights:
        if not args.config:
            print("--random_weights needs --config", file=sys.stderr)
            return 2
        import torch
        from pytriton_llama_b200.weights import write_random_model
        write_random_model(args.random_weights, json.loads(Path(args.config).read_text()), seed=args.seed,
                           dtype=torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
        args.checkpoints_dir = args.random_weights
    if not args.checkpoints_dir:
        print("give --checkpoints_dir or --random_weights", file=sys.stderr)
        return 2
    folder = Path(args.checkpoints_dir)
    from pytriton_llama_b200.engine.llm import GenerateStreamText
    generator = GenerateStreamText(
        checkpoints_dir=str(folder), tokenizer_path=str(folder) if _has_tokenizer(folder) else None,
        max_gpu_num_blocks=args.max_gpu_num_blocks, max_seq_len=args.max_seq_len,
        load_model=args.load_model, triton_weight=args.triton_weight, compiled_model=args.compiled_model,
        device=args.device, dtype=args.dtype, page_size=args.page_size, seed=args.seed, timing=args.stats)
    engine = generator.llm.engine
    if args.stats and engine.memory_report:
        print(f"[stats] cache pool: {json.dumps(engine.memory_report)}", file=sys.stderr)

    def show_stats() -> None:
        if args.stats:
            print(f"[stats] {json.dumps(engine.stats.summary())}", file=sys.stderr)

    def run_ids(ids: List[int]) -> None:
        for batch in generator.generate_stream([ids], args.max_gen_len, args.temperature, args.top_p):
            if batch[0]:
                print(" ".join(str(t) for t in batch[0]), end=" ", flush=True)
        print()
        show_stats()

    from pytriton_llama_b200.utils import prompt_for_tokenizer
    chat = prompt_for_tokenizer(generator.tokenizer, raw=args.raw_prompt, system=args.system)

    def run_text(text: str) -> None:
        shown = ""
        for completions in generator.text_completion_stream([chat.render(text)], args.temperature, args.top_p, args.max_gen_len):
            new = completions[0]["generation"][len(shown):]
            shown = completions[0]["generation"]
            print(new, end="", flush=True)
        print()
        chat.record(shown)
        show_stats()

    if args.prompt_ids:
        run_ids(args.prompt_ids)
        return 0
    if args.prompt is not None:
        run_text(args.prompt)
        return 0
    text_mode = generator.tokenizer is not None
    while True:
        try:
            line = input("prompt ('exit' to quit)" + ("" if text_mode else " as token ids") + ": ")
        except EOFError:
            break
        if line.strip().lower() == "exit":
            break
        if not line.strip():
            continue
        if text_mode:
            run_text(line)
        else:
            try:
                ids = [int(t) for t in line.replace(",", " ").split()]
            except ValueError:
                print("token ids must be integers", file=sys.stderr)
                continue
            run_ids(ids)
        print("\n==================================\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
