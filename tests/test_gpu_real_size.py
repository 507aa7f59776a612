"""The whole Llama-3.2-1B shape (16 layers, hidden 2,048, 32 query heads over 8 kv heads of size 64,
feed-forward width 8,192, vocabulary 128,256, llama3 rotary scaling by 32, tied head, pages of 16)
with seeded random weights, replayed in every cut against the plain implementation in float64.

The tiny configurations cannot show what only real sizes have: sums over 8,192 terms in the
float32 products, a 128,256-wide float32 head, rotation angles of positions in the thousands, 16
layers of accumulated rounding, block tables of many dozens of pages.  float32: every wanted row
within 1e-4 (absolute) of the oracle; bfloat16: the relative rule of the small tests.  The oracle
runs on the GPU through torch (it is the plain implementation of tests/plain_llama.py with its
tensors moved there; lite_llama's own whole-model check at real size is tests/test_LlamaModel.py:213-237).
"""
import gc
import json

import pytest
import torch

import plain_llama
import traces
from conftest import BF16_MAX_REL, BF16_MEAN_REL, FP32_TOL, random_tokens

pytestmark = pytest.mark.gpu

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256,
    "rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                              "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
PAGE = 16
LENGTHS = [40, 300, 700, 1100]         # every request but the first crosses many pages
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _seqs():
    return {f"r{i}": random_tokens(n, LLAMA_1B["vocab_size"], 7000 + i) for i, n in enumerate(LENGTHS)}


def _families(seqs):
    return {
        "whole": traces.whole(seqs),
        "prefill_then_decode": traces.prefill_then_decode(seqs, tail=32),
        "portions": traces.portions(seqs, sizes=(130, 2, 257, 33, 2, 64, 17, 300, 5, 96)),
        "mixed": traces.mixed(seqs, live=4, sizes=(97, 2, 160, 33, 2, 64), decode_tail=6),
    }


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def real_size(request, tmp_path_factory):
    """(compute type, model folder, request -> float64 oracle logits on the GPU).  The weights are
    drawn once with the package's device-side random mode, q and k projections scaled so that
    attention is far from uniform (as for the tiny configurations), and written as a model folder
    that both sides read with their own readers."""
    from pytriton_llama_b200.config.registry import resolve_architecture
    from pytriton_llama_b200.models.decoder import DecoderModel
    from pytriton_llama_b200.parts.base import Runtime
    from pytriton_llama_b200.weights import write_file
    from pytriton_llama_b200.weights.random_init import random_tensors_on_device
    dtype = request.param
    folder = tmp_path_factory.mktemp(f"llama_1b_{dtype}")
    arch = resolve_architecture(LLAMA_1B)
    spec = arch.spec_from_config(arch.config_from_dict(LLAMA_1B), norm_init="ones_jitter")
    expected = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32, ops=None)).expected_tensors()
    tensors = random_tensors_on_device(expected, 2024, 0.02, torch.float32, "cuda:0")
    gain = 2.0 if dtype == "float32" else 1.0
    for k in tensors:
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            tensors[k] = tensors[k] * gain
    tensors = {k: v.to(DTYPES[dtype]).cpu() for k, v in tensors.items()}
    (folder / "config.json").write_text(json.dumps(LLAMA_1B))
    write_file(folder / "model.safetensors", tensors)
    del tensors
    cfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    w = {k: v.cuda() for k, v in w.items()}
    with torch.no_grad():
        ref = {r: plain_llama.forward(cfg, w, s) for r, s in _seqs().items()}
    del w
    gc.collect()
    torch.cuda.empty_cache()
    yield dtype, folder, ref
    del ref
    (folder / "model.safetensors").unlink()
    gc.collect()
    torch.cuda.empty_cache()


def _replay_and_compare(engine, steps, ref, dtype, what):
    """Replays on the device and compares each step's wanted rows with the oracle's rows there."""
    from pytriton_llama_b200.engine.engine import StepEntry
    fed = {}
    worst, worst_at, total, count = 0.0, None, 0.0, 0
    scale = max(1.0, max(float(v.abs().max()) for v in ref.values()))
    for s in steps:
        out = engine.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        row = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            if e["want"]:
                n = len(e["want"])
                idx = torch.tensor([base + w for w in e["want"]], device="cuda")
                got = out.logits[row:row + n].double()
                assert torch.isfinite(got).all(), (what, s["step"], e["id"])
                diff = (got - ref[e["id"]].index_select(0, idx)).abs()
                m = float(diff.max())
                if m > worst:
                    worst, worst_at = m, (s["step"], e["id"], base + e["want"][int(diff.max(dim=1).values.argmax())])
                total += float(diff.sum())
                count += diff.numel()
                row += n
            fed[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            engine.finish(rid)
            fed.pop(rid, None)
        engine.cache.check_invariants()
    if dtype == "float32":
        assert worst < FP32_TOL, f"{what}: max |diff| {worst:.3e} at (step, request, position) {worst_at}"
    else:
        assert worst < BF16_MAX_REL * scale, f"{what}: max |diff| {worst:.3e} (scale {scale:.2f}) at {worst_at}"
        assert total / count < BF16_MEAN_REL * scale, f"{what}: mean |diff| {total / count:.3e} (scale {scale:.2f})"
    return worst


def test_full_llama_1b_shape_in_every_cut(real_size):
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.engine import Engine
    dtype, folder, ref = real_size
    seqs = _seqs()
    families = _families(seqs)
    pages = {name: -(-traces.max_live_tokens(steps, PAGE) // PAGE) for name, steps in families.items()}
    engine, engine_pages = None, 0
    report = {}
    for name, steps in families.items():
        # one engine per pool size: the pool holds exactly what the trace needs, so pages are used again
        if engine is None or engine_pages != pages[name]:
            engine_pages = pages[name]
            del engine
            gc.collect()
            torch.cuda.empty_cache()
            engine = Engine(folder, EngineConfig(dtype=dtype, page_size=PAGE, max_gpu_num_blocks=pages[name], max_seq_len=1152,
                                                 max_num_seqs=4, max_batched_tokens=2048), device="cuda:0")
        report[name] = _replay_and_compare(engine, steps, ref, dtype, f"{dtype} {name}")
        assert engine.cache.free_pages() == pages[name]
        engine.check_device_status()
    print(f"\nLlama-3.2-1B shape, {dtype}: max |logit difference| per cut {report}")
