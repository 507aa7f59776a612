"""The step function's host side (batch assembly, positions, block tables, page reuse) without a
GPU: the engine runs with the plain PyTorch operator set of tests/torch_ops.py in place of the CUDA
kernels and must reproduce the whole-sequence plain implementation for every way of cutting."""
import pytest
import torch

import plain_llama
import traces
from conftest import FP32_TOL, PAGE_SIZE, TINY, random_tokens
from torch_ops import TorchOps
from pytriton_llama_b200.cache.manager import OutOfPages
from pytriton_llama_b200.config import EngineConfig
from pytriton_llama_b200.engine.engine import Engine, StepEntry


def _engine(folder, name, pages, max_seq_len=256):
    cfg = EngineConfig(dtype="float32", page_size=PAGE_SIZE[name], max_gpu_num_blocks=pages, max_seq_len=max_seq_len,
                       max_num_seqs=4)
    return Engine(folder, cfg, device="cpu", ops=TorchOps())


@pytest.mark.parametrize("name", ["A", "B"])
def test_every_cut_gives_the_whole_sequence_logits(model_folders, name):
    folder = model_folders(name)
    cfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    vocab = TINY[name]["vocab_size"]
    lens = {"A": [5, 11, 17, 40, 23], "B": [1, 9, 33, 70, 12]}[name]
    seqs = {f"r{i}": random_tokens(n, vocab, 100 + i) for i, n in enumerate(lens)}
    ref = {r: plain_llama.forward(cfg, w, s) for r, s in seqs.items()}
    for family in (traces.whole, traces.prefill_then_decode, traces.portions, traces.mixed):
        steps = family(seqs)
        pages = -(-traces.max_live_tokens(steps, PAGE_SIZE[name]) // PAGE_SIZE[name])
        eng = _engine(folder, name, pages)
        got = traces.replay(eng, steps)
        for r in seqs:
            assert (got[r].double() - ref[r]).abs().max() < FP32_TOL, (family.__name__, r)
        assert eng.cache.free_pages() == pages and eng.cache.free_slots() == 4


def test_step_refuses_bad_input_and_leaves_the_cache_alone(model_folders):
    eng = _engine(model_folders("A"), "A", pages=4, max_seq_len=32)
    with pytest.raises(ValueError):
        eng.step([StepEntry("a", [1, 2, 999])])                     # outside the vocabulary
    with pytest.raises(ValueError):
        eng.step([StepEntry("a", [1, 2], want=[2])])                # wants a place it did not bring
    with pytest.raises(ValueError):
        eng.step([StepEntry("a", [1]), StepEntry("a", [2])])        # one request twice
    with pytest.raises(ValueError):
        eng.step([StepEntry("a", list(range(33)))])                 # longer than max_seq_len
    with pytest.raises(OutOfPages):
        eng.step([StepEntry("a", list(range(10))), StepEntry("b", list(range(10)))])   # 3 + 3 pages of 4
    assert eng.cache.free_pages() == 4 and not eng.cache.live_requests()
    out = eng.step([StepEntry("a", [1, 2, 3], want=[])])
    assert out.logits is None and out.num_tokens == 3
    out = eng.step([StepEntry("a", [4], want=[0]), StepEntry("b", [], want=[])])
    assert out.logits.shape == (1, 256) and out.rows == [("a", 0)]
