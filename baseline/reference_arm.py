"""The reference arm of bench.py: lite_llama itself, unmodified, on the benchmark's shape.

``run(args)`` drives lite_llama's stock entry point ``GenerateText.generate(prompt_tokens,
max_gen_len, temperature, top_p)`` (lite_llama/generate.py:87-154) on a Llama-3.2-1B-shaped model
with random float16 weights: batch 8, contexts that end at 4,096 tokens, the same number of decode
steps as the other arm.  Nothing of this repository's engine or kernel library is imported here.

lite_llama is a plain package tree without setup.py / pyproject.toml, so it is copied (not pip
installed) into ``baseline/_ref/lite_llama`` and imported from there.  What its stock path needs
and this box lacks is supplied from outside, without touching its files:

* ``accelerate`` is not installed; lite_llama/executor/model_executor.py:6 imports it for
  ``init_empty_weights`` (:97), which only has to be a context manager around the model's
  construction.  A two-function module of that name is put into ``sys.modules``.
* ``lite_llama/__init__.py`` imports the LLaVA path (PIL, requests, ...); a bare package object
  with the right ``__path__`` stands in for it so that ``lite_llama.generate`` imports alone.
* a checkpoint folder in lite_llama's own layout: ``config.json`` (HF keys plus ``max_seq_len``),
  one ``*.pth`` state dict in the names that lite_llama/executor/weight_convert.py:193-246 produces
  (k|v fused as ``kv_proj_weight``), and a minimal tokenizer folder built offline (the loop needs
  its pad / eos ids only, lite_llama/generate.py:113,146).

Decode time per step is the difference of two ``generate`` calls that differ in ``max_gen_len``
by K steps (CUDA events around each call), so that the prefill, which both calls do, cancels.
"""
from __future__ import annotations

import contextlib
import io
import json
import os
import shutil
import statistics
import sys
import tempfile
import time
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
REFERENCE_SOURCE = Path(os.environ.get("PTL_REFERENCE_SOURCE", "/root/reference"))     # the lite_llama checkout to copy from


class ReferenceUnavailable(RuntimeError):
    pass


def ensure_reference_copy() -> Path:
    """``baseline/_ref/lite_llama``, copied from the reference checkout when it is not there yet."""
    pkg = REF_DIR / "lite_llama"
    if (pkg / "generate.py").is_file():
        return REF_DIR
    src = REFERENCE_SOURCE / "lite_llama"
    if not src.is_dir():
        raise ReferenceUnavailable(f"{pkg} is missing and there is no reference checkout at {REFERENCE_SOURCE} to copy it from")
    REF_DIR.mkdir(parents=True, exist_ok=True)
    shutil.copytree(src, pkg, dirs_exist_ok=True)
    return REF_DIR


def import_generate():
    """lite_llama.generate (its GenerateText class), imported from the copy with the two stand-ins."""
    ref = ensure_reference_copy()
    if "accelerate" not in sys.modules:
        try:
            import accelerate  # noqa: F401
        except ImportError:
            import importlib.machinery
            import transformers  # noqa: F401  (looks for accelerate when first imported: let it see that there is none)
            shim = types.ModuleType("accelerate")
            shim.__spec__ = importlib.machinery.ModuleSpec("accelerate", None)

            @contextlib.contextmanager
            def init_empty_weights(*args, **kwargs):
                yield

            def load_checkpoint_and_dispatch(*args, **kwargs):
                raise NotImplementedError("accelerate is not installed; lite_llama's stock path does not call this")
            shim.init_empty_weights = init_empty_weights
            shim.load_checkpoint_and_dispatch = load_checkpoint_and_dispatch
            sys.modules["accelerate"] = shim
    pkg = types.ModuleType("lite_llama")
    pkg.__path__ = [str(ref / "lite_llama")]
    sys.modules["lite_llama"] = pkg
    import lite_llama.generate as generate
    return generate


def write_checkpoint(folder: Path, cfg: dict, max_seq_len: int, seed: int = 0) -> None:
    """config.json + model.pth (random float16, lite_llama's names) + tokenizer files."""
    import torch
    folder.mkdir(parents=True, exist_ok=True)
    stored = dict(cfg, max_seq_len=max_seq_len, torch_dtype="float16", eos_token_id=1, bos_token_id=2)
    (folder / "config.json").write_text(json.dumps(stored))
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = H // nq
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=dev).manual_seed(seed)

    def mat(*shape):
        return (0.02 * torch.randn(*shape, generator=gen, device=dev)).half().cpu()

    sd = {"embed_tokens.weight": mat(V, H), "norm_weight": torch.ones(H)}
    sd["lm_head.weight"] = sd["embed_tokens.weight"].clone()          # tied head: lite_llama keeps a copy
    for i in range(L):
        p = f"layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = mat(nq * d, H)
        sd[p + "self_attn.kv_proj_weight"] = mat(2 * nkv * d, H)
        sd[p + "self_attn.o_proj.weight"] = mat(H, nq * d)
        sd[p + "mlp.gate_proj.weight"] = mat(I, H)
        sd[p + "mlp.up_proj.weight"] = mat(I, H)
        sd[p + "mlp.down_proj.weight"] = mat(H, I)
        sd[p + "attention_norm_weight"] = torch.ones(H)
        sd[p + "ffn_norm_weight"] = torch.ones(H)
    torch.save(sd, folder / "model.pth")
    # the smallest tokenizer AutoTokenizer loads offline: three words, pad and eos named
    from tokenizers import Tokenizer, models, pre_tokenizers
    tok = Tokenizer(models.WordLevel({"<pad>": 0, "<eos>": 1, "<bos>": 2, "a": 3}, unk_token="<pad>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(str(folder / "tokenizer.json"))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<eos>", "pad_token": "<pad>", "bos_token": "<bos>",
         "unk_token": "<pad>", "model_max_length": max_seq_len}))
    (folder / "special_tokens_map.json").write_text(json.dumps(
        {"eos_token": "<eos>", "pad_token": "<pad>", "bos_token": "<bos>", "unk_token": "<pad>"}))


def run(model_cfg: dict, context: int, prefill_tokens: int, batch: int, steps: int, warmup: int, points, clock_sampler=None) -> dict:
    """The reference's numbers as a dict in the shape of bench.py's JSON line."""
    import torch
    generate_mod = import_generate()
    W, K = max(3, warmup), steps
    max_batch = max([batch] + list(points))
    gen = torch.Generator().manual_seed(0)
    vocab = model_cfg["vocab_size"]

    def prompts(n, length):
        return [torch.randint(4, vocab, (length,), generator=gen).tolist() for _ in range(n)]

    with tempfile.TemporaryDirectory(prefix="lite_llama_ckpt_") as tmp:
        folder = Path(tmp) / "llama-3.2-1b-random"
        write_checkpoint(folder, model_cfg, max_seq_len=context + 8)
        quiet = io.StringIO()          # the stock loop prints its cache indices every step (model_executor.py:311)
        with contextlib.redirect_stdout(quiet):
            g = generate_mod.GenerateText(checkpoints_dir=str(folder), tokenizer_path=str(folder), max_seq_len=context + 8,
                                          max_gpu_num_blocks=max_batch * (context + 8) + 64, load_model=True,
                                          triton_weight=True, compiled_model=False, device="cuda")

        def timed_generate(prompt_tokens, max_gen_len):
            """(device ms, wall s) of one stock generate call, tokens in from host lists, ids back to the host."""
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            quiet.seek(0)
            quiet.truncate()
            with contextlib.redirect_stdout(quiet):
                out = g.generate(prompt_tokens, max_gen_len=max_gen_len, temperature=0.6, top_p=0.9)
            ids = out.tolist()
            end.record()
            torch.cuda.synchronize()
            return start.elapsed_time(end), time.perf_counter() - t0, ids

        def decode_rate(b, k, sampler=None):
            """Decode steps k at batch b whose contexts end at `context`: two calls that differ by k steps."""
            ctx0 = context - k - W
            pr = prompts(b, ctx0)
            timed_generate(pr, 1 + 2)                                   # compiles the kernels for these shapes
            short_ms, short_s, _ = timed_generate(pr, 1 + W)
            if sampler is not None:
                with sampler as cs:
                    long_ms, long_s, _ = timed_generate(pr, 1 + W + k)
                clocks = cs.summary()
            else:
                long_ms, long_s, _ = timed_generate(pr, 1 + W + k)
                clocks = None
            return (long_ms - short_ms) / k, (long_s - short_s) / k, clocks

        ms_step, s_step, clocks = decode_rate(batch, K, clock_sampler)
        pts = {}
        for pb in points:
            ms, _, _ = decode_rate(pb, max(16, K // 2))
            pts[f"decode_b{pb}"] = round(pb / ms * 1e3, 1)
        pr = prompts(1, prefill_tokens)
        timed_generate(pr, 1)
        pf = [timed_generate(pr, 1)[0] for _ in range(3)]
        prefill_ms = statistics.median(pf)

    return {
        "metric": "decode_tokens_per_s", "value": round(batch / ms_step * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K,
        "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic", "impl": "reference",
        "config": {"model": "Llama-3.2-1B shape, random weights", "layers": model_cfg["num_hidden_layers"],
                   "hidden": model_cfg["hidden_size"], "heads": model_cfg["num_attention_heads"],
                   "kv_heads": model_cfg["num_key_value_heads"], "intermediate": model_cfg["intermediate_size"], "vocab": vocab,
                   "global_batch": batch, "seq_len": context, "parallelism": "single-gpu",
                   "api": "lite_llama GenerateText.generate, stock path, temperature 0.6 top_p 0.9",
                   "timing": "difference of two generate calls that differ by K decode steps"},
        "clocks": clocks,
        "e2e": {"value": round(batch / s_step, 1), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "ms_per_step": round(s_step * 1e3, 4),
                "note": "prompt ids go up once per generate call and the ids come back once at its end; the stock loop syncs every step"},
        "gpu_launches": None,
        "prefill": {"value": round(prefill_tokens / prefill_ms * 1e3, 1), "tokens": prefill_tokens, "ms": round(prefill_ms, 3),
                    "note": "one generate call of one 2,048-token prompt and one sampled token"},
        "points": pts,
    }
