"""Replay of the same requests cut in every way, in float32 and bfloat16, against the plain
whole-sequence implementation (GPU)."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import traces
from conftest import PAGE_SIZE, ROOT, TINY, random_tokens
from gpu_common import assert_close, make_engine, reference_logits, stored_dtype

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 11, 17, 90, 47, 130], "B": [1, 9, 33, 70, 150, 41], "C": [40, 3, 100, 77, 260, 18],
           "D": [70, 1, 200, 33, 129, 64], "E": [65, 140, 2, 90, 31, 128]}


def _seqs(name):
    vocab = TINY[name]["vocab_size"]
    return {f"{name}{i}": random_tokens(n, vocab, 1000 + 17 * i + len(name)) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def references(model_folders):
    cache = {}

    def get(name, dtype):
        key = (name, dtype)
        if key not in cache:
            cache[key] = reference_logits(model_folders(name, stored_dtype(dtype)), _seqs(name))
        return cache[key]
    return get


FAMILIES = {
    "whole": traces.whole,
    "prefill_then_decode": traces.prefill_then_decode,
    "portions": traces.portions,
    "mixed": traces.mixed,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("family", list(FAMILIES))
def test_logits_do_not_depend_on_the_cut(model_folders, references, name, dtype, family):
    seqs = _seqs(name)
    ref = references(name, dtype)
    steps = FAMILIES[family](seqs)
    ps = PAGE_SIZE[name]
    pages = -(-traces.max_live_tokens(steps, ps) // ps)       # exactly what the trace needs: pages are used again
    eng = make_engine(model_folders(name, stored_dtype(dtype)), name, dtype, pages)
    got = traces.replay(eng, steps)
    for r in seqs:
        assert_close(got[r], ref[r], dtype, f"{family} {r}")
    assert eng.cache.free_pages() == pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_decode_steps_from_cuda_graphs(model_folders, references, name, dtype):
    """With ``compiled_model`` single-token steps replay captured graphs of padded batch sizes
    (1, 2, 4): the logits are those of the plain implementation all the same, also when the batch
    shrinks and grows and a prompt portion interrupts the decoding."""
    seqs = _seqs(name)
    ref = references(name, dtype)
    steps = traces.mixed(seqs, live=3, sizes=(40, 23, 64), decode_tail=30)
    ps = PAGE_SIZE[name]
    pages = -(-traces.max_live_tokens(steps, ps) // ps)
    eng = make_engine(model_folders(name, stored_dtype(dtype)), name, dtype, pages, compiled_model=True)
    got = traces.replay(eng, steps)
    assert set(eng._graphs) >= {1, 2, 4}
    for r in seqs:
        assert_close(got[r], ref[r], dtype, f"graph {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(model_folders, references, dtype):
    """Positions 0, 1, 2 each as a step of their own, and a request that is one token long."""
    name = "B"
    seqs = _seqs(name)
    ref = references(name, dtype)
    eng = make_engine(model_folders(name, stored_dtype(dtype)), name, dtype, pages=8)
    from pytriton_llama_b200.engine.engine import StepEntry
    r = "B3"
    for p in range(3):
        out = eng.step([StepEntry(r, [seqs[r][p]], [0])])
        assert_close(out.logits, ref[r][p:p + 1], dtype, f"position {p}")
    out = eng.step([StepEntry("B0", seqs["B0"], [0]), StepEntry(r, seqs[r][3:5], [1])])
    assert_close(out.logits[0:1], ref["B0"][0:1], dtype, "one-token request")
    assert_close(out.logits[1:2], ref[r][4:5], dtype, "position 4 beside it")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_folders, dtype):
    """A short prompt, then 400 tokens one by one across many pages, beside a second request."""
    name = "A"
    vocab = TINY[name]["vocab_size"]
    seqs = {"long": random_tokens(420, vocab, 5), "side": random_tokens(300, vocab, 6)}
    ref = reference_logits(model_folders(name, stored_dtype(dtype)), seqs)
    eng = make_engine(model_folders(name, stored_dtype(dtype)), name, dtype, pages=190, max_seq_len=512)
    from pytriton_llama_b200.engine.engine import StepEntry
    out = eng.step([StepEntry("long", seqs["long"][:20], [19]), StepEntry("side", seqs["side"][:7], [])])
    rows = {"long": [out.logits[0].cpu()], "side": []}
    for p in range(20, 420):
        entries = [StepEntry("long", [seqs["long"][p]], [0])]
        q = 7 + (p - 20)
        if q < 300:
            entries.append(StepEntry("side", [seqs["side"][q]], [0]))
        out = eng.step(entries)
        rows["long"].append(out.logits[0].cpu())
        if q < 300:
            rows["side"].append(out.logits[1].cpu())
    assert_close(torch.stack(rows["long"]), ref["long"][19:], dtype, "long")
    assert_close(torch.stack(rows["side"]), ref["side"][7:], dtype, "side")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_graphs_captured_per_class_of_context_length(model_folders, dtype):
    """With ``compiled_model`` a step of single tokens replays the graph captured for its batch size
    and for the class its longest context falls into (here up to 64, up to 128, and the engine's 512):
    300 tokens one by one through all three classes, beside a second request that ends on the way."""
    from pytriton_llama_b200.engine.engine import StepEntry, _DecodeShape
    name = "A"
    vocab = TINY[name]["vocab_size"]
    seqs = {"long": random_tokens(330, vocab, 7), "side": random_tokens(90, vocab, 8)}
    ref = reference_logits(model_folders(name, stored_dtype(dtype)), seqs)
    eng = make_engine(model_folders(name, stored_dtype(dtype)), name, dtype, pages=190, max_seq_len=512, compiled_model=True,
                      graph_context_buckets=(64, 128))
    out = eng.step([StepEntry("long", seqs["long"][:30], [29]), StepEntry("side", seqs["side"][:5], [])])
    rows = {"long": [out.logits[0].cpu()], "side": []}
    for p in range(30, 330):
        entries = [StepEntry("long", [seqs["long"][p]], [0])]
        q = 5 + (p - 30)
        if q < 90:
            entries.append(StepEntry("side", [seqs["side"][q]], [0]))
        out = eng.step(entries)
        rows["long"].append(out.logits[0].cpu())
        if q < 90:
            rows["side"].append(out.logits[1].cpu())
        if q == 89:
            eng.finish("side")
    assert set(eng._graphs) >= {_DecodeShape(2, 64), _DecodeShape(2, 128), _DecodeShape(1, 128), 1}
    assert_close(torch.stack(rows["long"]), ref["long"][29:], dtype, "long")
    assert_close(torch.stack(rows["side"]), ref["side"][5:], dtype, "side")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_folders, references, tmp_path, dtype):
    """bin/trace_run as a user runs it: JSON steps on standard input, <step>.f32 files out."""
    name = "B"
    seqs = _seqs(name)
    ref = references(name, dtype)
    steps = traces.mixed(seqs)
    for s in steps[::3]:                       # some steps want nothing, some only a few places
        for e in s["entries"]:
            e["want"] = e["want"][-1:]
    steps[1]["entries"][0]["want"] = []
    out_dir = tmp_path / "out"
    n = traces.max_live_tokens(steps, 64)
    proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(model_folders(name, stored_dtype(dtype))),
                           "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(n)],
                          input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {s['step']}" for s in steps]
    vocab = TINY[name]["vocab_size"]
    fed = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out_dir / f"{s['step']}.f32"
        if not wanted:
            assert not path.exists()
            for e in s["entries"]:
                fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
            continue
        data = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(wanted, vocab))
        row = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                assert_close(data[row:row + 1], ref[e["id"]][base + w:base + w + 1], dtype, f"step {s['step']} {e['id']}[{base + w}]")
                row += 1
            fed[e["id"]] = base + len(e["tokens"])
