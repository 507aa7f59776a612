"""Random traces through the engine against the plain implementation: random cuts, live sets and
skipped steps, wanted places chosen at random, pools with exactly the pages a trace needs or a few
more, captured steps on and off (with several layouts of their context classes), both compute
types, all tiny configurations (the five of the other tests and seven more with head sizes of 80 to
256, large and trivial groups, odd widths).  Every seed is one trace; a failure names its seed."""
import random

import pytest
import torch

import traces
from conftest import PAGE_SIZE, TINY, random_tokens
from gpu_common import assert_close, make_engine, reference_logits, stored_dtype

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("block", range(10))
def test_random_traces(model_folders, block):
    for seed in range(block * 12, block * 12 + 12):
        rng = random.Random(seed)
        name = rng.choice(sorted(TINY))
        dtype = rng.choice(["float32", "bfloat16"])
        folder = model_folders(name, stored_dtype(dtype))
        vocab = TINY[name]["vocab_size"]
        seqs = {f"r{i}": random_tokens(rng.choice([1, 2, 3, 17, 40, 64, 65, 130, 257, 300, 420]), vocab, seed * 100 + i)
                for i in range(rng.randint(2, 7))}
        steps = traces.random_trace(seqs, rng, live=rng.randint(1, 4))
        ps = PAGE_SIZE[name]
        pages = -(-traces.max_live_tokens(steps, ps) // ps) + rng.choice([0, 0, 1, 5])
        eng = make_engine(folder, name, dtype, pages, max_seq_len=512, compiled_model=rng.random() < 0.6,
                          graph_context_buckets=rng.choice([(64, 128), (4096, 16384, 65536), (32,)]))
        got = traces.replay(eng, steps)
        ref = reference_logits(folder, seqs)
        for r in seqs:
            wanted = traces.wanted_positions(steps, r)
            if wanted:
                assert_close(got[r], ref[r][wanted], dtype, f"seed {seed}: {name} {dtype} {r}")
        assert eng.cache.free_pages() == pages, f"seed {seed}"
        eng.check_device_status()
