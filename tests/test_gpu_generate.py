"""Generation through the Python entry points and the command line: greedy tokens against the
plain implementation, seeded sampling, and scheduling under page pressure (GPU)."""
import subprocess
import sys

import pytest
import torch

import plain_llama
from conftest import PAGE_SIZE, ROOT, TINY, random_tokens
from gpu_common import stored_dtype

pytestmark = pytest.mark.gpu


def _llm(folder, name, dtype, pages, **extra):
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.llm import LLM
    cfg = EngineConfig(dtype=dtype, page_size=PAGE_SIZE[name], max_gpu_num_blocks=pages, max_seq_len=extra.pop("max_seq_len", 128),
                       max_num_seqs=extra.pop("max_num_seqs", 4), max_batched_tokens=extra.pop("max_batched_tokens", 16), **extra)
    return LLM(folder, cfg)


def _plain_greedy(folder, prompts, n, stop=()):
    cfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    return [plain_llama.greedy_generate(cfg, w, p, n, stop_ids=stop) for p in prompts]


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_float32_equals_plain(model_folders, name):
    """The tiny models' generation workload: prompts of 5/11/17 (A) and 1/9/33/70 (B) tokens, 8 new tokens each."""
    from pytriton_llama_b200.sampling import SamplingParams
    folder = model_folders(name)
    vocab = TINY[name]["vocab_size"]
    lens = {"A": [5, 11, 17], "B": [1, 9, 33, 70]}[name]
    prompts = [random_tokens(n, vocab, 300 + n) for n in lens]
    eos = TINY[name]["eos_token_id"]
    stop = [eos] if isinstance(eos, int) else list(eos)
    want = _plain_greedy(folder, prompts, 8, stop)
    llm = _llm(folder, name, "float32", pages=60)
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_gen_len=8))
    assert got == want
    assert llm.engine.cache.free_pages() == 60
    # the same through lite_llama's class names
    from pytriton_llama_b200 import GenerateStreamText, GenerateText
    gen = GenerateText(str(folder), None, max_seq_len=128, max_gpu_num_blocks=60, dtype="float32", page_size=PAGE_SIZE[name])
    out = gen.generate(prompts, max_gen_len=8, temperature=0.0)
    trimmed = [w[: next((i for i, t in enumerate(w) if t in stop), len(w))] for w in want]
    assert out == trimmed
    assert gen.generate(prompts[:1], max_gen_len=8, temperature=0.0, echo=True) == [prompts[0] + trimmed[0]]
    # log-probabilities of the generated tokens, as lite_llama's logprobs variant reports them
    toks, lps = gen.generate(prompts, max_gen_len=8, temperature=0.0, logprobs=True)
    assert toks == trimmed
    cfg64, w64 = plain_llama.load_model_folder(folder, dtype=torch.float64)
    for p_, out_, lp_ in zip(prompts, toks, lps):
        assert len(lp_) == len(out_)
        if out_:
            ref_lp = torch.log_softmax(plain_llama.forward(cfg64, w64, p_ + out_), -1)
            for i, (tok, got_lp) in enumerate(zip(out_, lp_)):
                assert abs(got_lp - float(ref_lp[len(p_) + i - 1, tok])) < 2e-4
    stream = GenerateStreamText(str(folder), None, max_gpu_num_blocks=60, max_seq_len=128, dtype="float32", page_size=PAGE_SIZE[name])
    pieces = [[] for _ in prompts]
    for batch in stream.generate_stream(prompts, max_gen_len=8, temperature=0.0):
        for i, new in enumerate(batch):
            pieces[i] += new
    assert pieces == trimmed


def test_greedy_generation_bfloat16(model_folders):
    """bfloat16 may pick another token where two logits nearly tie; every picked token must be
    within rounding of the best logit of the plain model fed with the same history."""
    from pytriton_llama_b200.sampling import SamplingParams
    name = "B"
    folder = model_folders(name, torch.bfloat16)
    cfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    prompts = [random_tokens(n, 384, 400 + n) for n in (9, 33, 70)]
    llm = _llm(folder, name, "bfloat16", pages=60, compiled_model=True)     # overlapped steps, captured decode graphs
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_gen_len=8, stop_token_ids=[]))
    agree = 0
    for p, out in zip(prompts, got):
        assert 1 <= len(out) <= 8
        logits = plain_llama.forward(cfg, w, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - 0.04 * float(logits.abs().max()), (i, tok)
            agree += int(tok == int(row.argmax()))
    assert agree >= 0.8 * sum(len(o) for o in got)


def test_sampling_is_seeded_and_independent_of_batching(model_folders):
    """Temperature 0.8 from a fixed seed (configuration B): the float32 engine draws exactly the
    tokens the plain implementation draws from the same uniform numbers, whether the requests run
    together in portions of 16 or one at a time."""
    from pytriton_llama_b200.sampling import SamplingParams, uniform
    name = "B"
    folder = model_folders(name)
    cfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    prompts = [random_tokens(n, 384, 500 + n) for n in (1, 9, 33, 70)]
    params = SamplingParams(temperature=0.8, top_p=0.9, max_gen_len=6, stop_token_ids=[])
    llm = _llm(folder, name, "float32", pages=60, seed=1234)
    got = llm.generate(prompts, params)
    for number, (p, out) in enumerate(zip(prompts, got)):
        seq = list(p)
        for i, tok in enumerate(out):
            row = plain_llama.forward(cfg, w, seq)[-1]
            want = plain_llama.sample_token(row, 0.8, 0.9, uniform(1234, number, i))
            if tok != want:   # only a draw within rounding of a boundary of the distribution may differ
                pr = torch.softmax(row / 0.8, -1)
                keep = plain_llama.top_p_keep_mask(pr, 0.9)
                assert keep[tok]
                kept = torch.where(keep, pr, torch.zeros_like(pr))
                cdf = torch.cumsum(kept, 0) / kept.sum()
                u = uniform(1234, number, i)
                assert float(cdf[tok] - kept[tok] / kept.sum()) - 1e-5 <= u <= float(cdf[tok]) + 1e-5
            if tok in (382, 383):
                break
            seq.append(tok)
    llm2 = _llm(folder, name, "float32", pages=60, seed=1234, max_num_seqs=1)
    assert llm2.generate(prompts, params) == got
    llm3 = _llm(folder, name, "float32", pages=60, seed=99)
    assert llm3.generate(prompts, params) != got


def test_generation_under_page_pressure_preempts_and_still_matches(model_folders):
    """So few pages that running requests must give way and recompute: the tokens do not change."""
    from pytriton_llama_b200.sampling import SamplingParams
    name = "A"
    folder = model_folders(name)
    prompts = [random_tokens(n, 256, 600 + n) for n in (17, 11, 5, 14, 9)]
    want = _plain_greedy(folder, prompts, 12, [255])
    llm = _llm(folder, name, "float32", pages=14, max_batched_tokens=8)   # 56 tokens of cache for 5 requests of up to 29
    reqs = [llm.add_request(p, SamplingParams(temperature=0.0, max_gen_len=12)) for p in prompts]
    steps = 0
    while llm.has_work():
        llm.step()
        llm.engine.cache.check_invariants()
        steps += 1
        assert steps < 400
    assert [r.output for r in reqs] == want
    assert sum(r.preemptions for r in reqs) > 0
    assert llm.engine.cache.free_pages() == 14
    too_big = llm.add_request(random_tokens(60, 256, 1), SamplingParams(temperature=0.0, max_gen_len=4))
    while llm.has_work():
        llm.step()
    assert too_big.finish_reason == "cache_too_small"


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("float32", "B")])
def test_overlapped_steps_and_captured_graphs_change_no_token(model_folders, dtype, name):
    """The next step launched before the last one's tokens are read (tokens handed over on the
    device), with and without captured decode graphs, roomy and under page pressure: the same
    tokens and finish reasons as stepping one at a time.  Stop tokens are ones that do occur."""
    from pytriton_llama_b200.sampling import SamplingParams
    folder = model_folders(name, stored_dtype(dtype))
    vocab = TINY[name]["vocab_size"]
    prompts = [random_tokens(n, vocab, 800 + n) for n in (17, 3, 29, 8, 12, 21)]
    ps = PAGE_SIZE[name]
    base = _llm(folder, name, dtype, pages=80, overlap_steps=False).generate(
        prompts, SamplingParams(temperature=0.0, max_gen_len=14, stop_token_ids=[]))
    stops = sorted({o[6] for o in base[:3]})
    settings = [SamplingParams(temperature=0.0, max_gen_len=14, stop_token_ids=stops),
                SamplingParams(temperature=0.7, top_p=0.9, max_gen_len=10, stop_token_ids=stops[:1], seed=5)]
    for pages in (80, -(-(29 + 14) // ps) + 3):
        for sp in settings:
            runs = []
            for overlap, graphs in ((False, False), (True, False), (True, True)):
                llm = _llm(folder, name, dtype, pages=pages, overlap_steps=overlap, compiled_model=graphs)
                reqs = [llm.add_request(p, sp) for p in prompts]
                for _ in llm.run():
                    pass
                llm.engine.check_device_status()
                llm.engine.cache.check_invariants()
                assert llm.engine.cache.free_pages() == pages
                runs.append(([list(r.output) for r in reqs], [r.finish_reason for r in reqs]))
            assert runs[0] == runs[1] == runs[2], (pages, sp)
            if sp.temperature == 0.0:
                assert any(r == "stop" for r in runs[0][1])


def test_command_line(model_folders, tmp_path):
    folder = model_folders("A")
    prompt = random_tokens(7, 256, 700)
    want = _plain_greedy(folder, [prompt], 5, [255])[0]
    want = want[: next((i for i, t in enumerate(want) if t == 255), len(want))]
    base = [sys.executable, str(ROOT / "cli.py"), "--checkpoints_dir", str(folder), "--dtype", "float32", "--temperature", "0",
            "--max_gen_len", "5", "--max_seq_len", "64", "--max_gpu_num_blocks", "16", "--page_size", "4"]
    out = subprocess.run(base + ["--prompt_ids"] + [str(t) for t in prompt], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert [int(t) for t in out.stdout.split()] == want
    # the prompt loop: token ids on standard input, 'exit' ends it
    loop = subprocess.run(base, input=" ".join(str(t) for t in prompt) + "\nexit\n", capture_output=True, text=True, timeout=600)
    assert loop.returncode == 0, loop.stderr[-2000:]
    assert " ".join(str(t) for t in want) in loop.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_steps_of_mixed_shapes_give_the_same_logits(model_folders, dtype):
    """Steps that hold prompt portions run from captured graphs of padded shapes once a shape has
    come twice.  The same steps (portions beside single tokens, three live requests, shapes that
    repeat and a step that wants two rows of one request) with and without captured graphs must
    agree, and the second engine must really have captured mixed shapes."""
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.engine import Engine, StepEntry
    folder = model_folders("B", stored_dtype(dtype))
    vocab = TINY["B"]["vocab_size"]
    prompts = {"a": random_tokens(150, vocab, 1), "b": random_tokens(90, vocab, 2), "c": random_tokens(40, vocab, 3)}
    steps = []
    for i in range(5):
        entries = [("a", prompts["a"][30 * i:30 * (i + 1)], [29])]
        if i >= 2:
            entries.append(("b", prompts["b"][30 * (i - 2):30 * (i - 1)], [0, 29] if i == 3 else [29]))
        if i >= 1:
            lo = 11 * (i - 1)
            entries.append(("c", prompts["c"][lo:lo + (1 if i % 2 else 10)], [0]))
        steps.append(entries)
    outs = {}
    for compiled in (False, True):
        cfg = EngineConfig(dtype=dtype, page_size=PAGE_SIZE["B"], max_gpu_num_blocks=64, max_seq_len=256, max_num_seqs=4,
                           max_batched_tokens=256, compiled_model=compiled, seed=0)
        eng = Engine(folder, cfg)
        res = []
        for _ in range(3):                         # the whole sequence three times: every shape has come before
            for entries in steps:
                out = eng.step([StepEntry(r, t, w) for r, t, w in entries])
                res.append(out.logits.float().cpu())
            eng.finish_all()
        eng.check_device_status()
        outs[compiled] = res
        if compiled:
            shapes = [k for k in eng._graphs if isinstance(k, tuple)]
            assert len(shapes) >= 3, shapes
    for a, b in zip(outs[False], outs[True]):
        assert a.shape == b.shape
        top = float(a.abs().max())
        assert float((a - b).abs().max()) <= (1e-5 if dtype == "float32" else 0.03) * top


@pytest.mark.parametrize("own_products", [False, True])
@pytest.mark.parametrize("hidden, heads, kv_heads, head_dim, inter", [(2048, 32, 8, 64, 8192), (3072, 24, 8, 128, 8192)])
def test_one_layer_of_real_widths_in_bfloat16(tmp_path, hidden, heads, kv_heads, head_dim, inter, own_products):
    """The tiny configurations never reach the kernels' paths for real widths: products of 2,048-wide
    rows with a few hundred and with more than a thousand tokens (parts of the K range, wide tiles on
    pairs of blocks), 32 query heads over 8 kv heads or 24 over 8 with head size 128, prompts of many
    key tiles.  One layer of the Llama-3.2-1B and -3B widths with a smaller vocabulary: a 1,400-token prompt in portions of 300 and 1,100
    (the first as a captured shape the second time round), then single tokens, against the plain
    implementation.  Once as the engine runs (products of many tokens and few tiles go to the library)
    and once with every product on this library's own tensor-core kernel (``own_products``: also the
    q|k|v projection that rotates and writes the cache in its epilogue, and the add epilogues)."""
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.engine import Engine, StepEntry
    from pytriton_llama_b200.weights.random_init import write_random_model
    config = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 1, "hidden_size": hidden,
        "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter, "vocab_size": 32064,
        "rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                                  "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
    }
    folder = write_random_model(tmp_path / "wide", config, seed=5, dtype=torch.bfloat16)
    prompt = random_tokens(1400, config["vocab_size"], 6)
    tail = random_tokens(6, config["vocab_size"], 7)
    cfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    ref = plain_llama.forward(cfg, w, prompt + tail)
    ecfg = EngineConfig(dtype="bfloat16", page_size=16, max_gpu_num_blocks=200, max_seq_len=1536, max_num_seqs=2,
                        max_batched_tokens=2048, compiled_model=True, seed=0)
    eng = Engine(folder, ecfg)
    eng.ops.library_products = not own_products
    from gpu_common import assert_close
    for attempt in range(2):                     # the second time the 300-token step runs from its captured graph
        out = eng.step([StepEntry("r", prompt[:300], [299])])
        assert_close(out.logits, ref[[299]], "bfloat16", f"portion of 300, attempt {attempt}")
        out = eng.step([StepEntry("r", prompt[300:], [0, 747, 1099])])
        assert_close(out.logits, ref[[300, 1047, 1399]], "bfloat16", f"portion of 1,100, attempt {attempt}")
        for i, t in enumerate(tail):
            out = eng.step([StepEntry("r", [t], [0])])
            assert_close(out.logits, ref[[1400 + i]], "bfloat16", f"single token {i}, attempt {attempt}")
        eng.finish("r")
    eng.check_device_status()
    assert any(isinstance(k, tuple) for k in eng._graphs)


def test_requests_that_arrive_while_others_decode(model_folders):
    """New prompts join while earlier requests generate, so most steps hold portions beside single
    tokens, in shapes that repeat: stepping one at a time without graphs and overlapped steps from
    captured graphs (single-token batches and mixed shapes) give the same tokens."""
    from pytriton_llama_b200.sampling import SamplingParams
    name, dtype = "B", "float32"
    folder = model_folders(name, stored_dtype(dtype))
    vocab = TINY[name]["vocab_size"]
    prompts = [random_tokens(n, vocab, 900 + i) for i, n in enumerate((23, 40, 9, 31, 18, 44, 12, 27, 35, 5))]
    sp = SamplingParams(temperature=0.0, max_gen_len=20, stop_token_ids=[])
    runs = []
    for overlap, graphs in ((False, False), (True, True)):
        llm = _llm(folder, name, dtype, pages=120, overlap_steps=overlap, compiled_model=graphs, max_num_seqs=8,
                   max_batched_tokens=24)
        reqs = [llm.add_request(p, sp) for p in prompts[:2]]
        waiting = list(prompts[2:])
        steps = 0
        while True:
            for _ in llm.run():
                steps += 1
                if waiting and steps % 3 == 0:
                    reqs.append(llm.add_request(waiting.pop(0), sp))
            if not waiting:
                break
            reqs.append(llm.add_request(waiting.pop(0), sp))
        llm.engine.check_device_status()
        llm.engine.cache.check_invariants()
        assert llm.engine.cache.free_pages() == 120
        if graphs:
            assert sum(isinstance(k, tuple) for k in llm.engine._graphs) >= 2
        runs.append({tuple(r.prompt): list(r.output) for r in reqs})
    assert runs[0] == runs[1]
    assert len(runs[0]) == len(prompts) and all(1 <= len(o) <= 20 for o in runs[0].values())


def _assert_tokens_within_rounding_of_plain(cfg, w, prompts, outputs, min_agree=0.8):
    """bfloat16 may pick another token where two logits nearly tie: every generated token must be
    within rounding of the best logit of the plain model fed with the same history."""
    agree = total = 0
    for p, out in zip(prompts, outputs):
        logits = plain_llama.forward(cfg, w, list(p) + list(out))
        top = float(logits.abs().max())
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - 0.04 * top, (len(p), i, tok)
            agree += int(tok == int(row.argmax()))
            total += 1
    assert agree >= min_agree * total, (agree, total)


@pytest.mark.parametrize("name", ["D", "E"])
def test_scheduler_on_the_bfloat16_tensor_core_path(model_folders, name):
    """The path the benchmark times, through the scheduler: head sizes 64 and 128 in bfloat16, so
    the tcgen05 prompt attention, the split-key decode attention with rotary encoding folded in,
    captured decode graphs and captured mixed shapes, the device-side hand-over of sampled tokens.
    Roomy and with so few pages that requests are pre-empted and recomputed, overlapped and one
    step at a time, with requests that arrive while others decode."""
    from pytriton_llama_b200.sampling import SamplingParams
    folder = model_folders(name, torch.bfloat16)
    cfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    vocab = TINY[name]["vocab_size"]
    ps = PAGE_SIZE[name]
    prompts = [random_tokens(n, vocab, 1200 + n) for n in (70, 9, 150, 33, 120, 17, 64, 200)]
    sp = SamplingParams(temperature=0.0, max_gen_len=24, stop_token_ids=[])
    roomy = 8 * -(-(200 + 24) // ps)
    tight = -(-(200 + 24) // ps) + 6                   # the longest request and a little more
    results = {}
    for pages in (roomy, tight):
        for overlap in (True, False):
            llm = _llm(folder, name, "bfloat16", pages=pages, max_seq_len=256, max_num_seqs=8, max_batched_tokens=64,
                       overlap_steps=overlap, compiled_model=True)
            reqs = [llm.add_request(p, sp) for p in prompts[:3]]
            waiting = list(prompts[3:])
            steps = 0
            while True:                                  # the others arrive while these decode
                for _ in llm.run():
                    steps += 1
                    if waiting and steps % 4 == 0:
                        reqs.append(llm.add_request(waiting.pop(0), sp))
                if not waiting:
                    break
                reqs.append(llm.add_request(waiting.pop(0), sp))
            llm.engine.check_device_status()
            llm.engine.cache.check_invariants()
            assert llm.engine.cache.free_pages() == pages
            assert all(len(r.output) == 24 and r.finish_reason == "length" for r in reqs)
            by_prompt = {tuple(r.prompt): list(r.output) for r in reqs}
            outs = [by_prompt[tuple(p)] for p in prompts]
            _assert_tokens_within_rounding_of_plain(cfg, w, prompts, outs)
            kinds = llm.engine._graphs
            assert any(isinstance(k, int) for k in kinds) and any(isinstance(k, tuple) for k in kinds)
            if pages == tight:
                assert sum(r.preemptions for r in reqs) > 0
            results[(pages, overlap)] = outs
    # with room for everybody the two modes plan the same steps, which run the same kernels: the same tokens
    assert results[(roomy, True)] == results[(roomy, False)]


@pytest.mark.parametrize("dtype, name", [("bfloat16", "D"), ("float32", "B")])
def test_more_mixed_shapes_than_captured_graphs_are_kept(model_folders, dtype, name):
    """Thirty different padded shapes, each stepped three times: the engine keeps at most 24
    captured graphs (the one used longest ago goes), all in one memory pool, captures evicted
    shapes again when they come back, and every step's logits equal those of an engine that
    captures nothing.  The logits handed out survive later steps."""
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.engine import Engine, StepEntry
    folder = model_folders(name, stored_dtype(dtype))
    vocab = TINY[name]["vocab_size"]
    lengths = [30, 100, 150, 200, 300, 400, 520, 650, 780, 900]
    plans = [(L, k) for L in lengths for k in (0, 1, 2)]            # a portion of L tokens beside k single tokens
    outs = {}
    for compiled in (False, True):
        cfg = EngineConfig(dtype=dtype, page_size=PAGE_SIZE[name], max_gpu_num_blocks=-(-1024 // PAGE_SIZE[name]) + 4,
                           max_seq_len=1024, max_num_seqs=4, max_batched_tokens=1024, compiled_model=compiled, seed=0)
        eng = Engine(folder, cfg)
        res, kept = [], []
        for rnd in range(3):
            for i, (L, k) in enumerate(plans):
                entries = [StepEntry("long", random_tokens(L, vocab, 3000 + i), [L - 1])]
                entries += [StepEntry(f"one{j}", random_tokens(1, vocab, 4000 + 10 * i + j), [0]) for j in range(k)]
                out = eng.step(entries)
                kept.append((out.logits, out.logits.clone()))
                res.append(out.logits.float().cpu())
                eng.finish_all()
        eng.check_device_status()
        for held, copy in kept:                                      # nothing that was handed out has been written again
            assert torch.equal(held, copy)
        if compiled:
            shapes = [g for g in eng._graphs if isinstance(g, tuple)]
            assert len(shapes) == eng.GRAPH_MAX_SHAPES == 24
            assert eng._shape_captures > 30                          # the six that had to go were captured again
        outs[compiled] = res
    for a, b in zip(outs[False], outs[True]):
        top = float(a.abs().max())
        assert float((a - b).abs().max()) <= (1e-5 if dtype == "float32" else 0.03) * top


def test_step_statistics_timers_and_a_pool_sized_from_free_memory(model_folders):
    """``max_gpu_num_blocks=None`` sizes the pool from the memory that is free after the weights
    (lite_llama/executor/mem_manager.py:98-108), capped at what the requests can ever hold; with
    ``timing`` every step reports its device time, the pages in use and milliseconds by class of
    kernels; generation works on such an engine."""
    from pytriton_llama_b200.config import EngineConfig
    from pytriton_llama_b200.engine.engine import Engine, StepEntry
    from pytriton_llama_b200.engine.llm import LLM
    from pytriton_llama_b200.sampling import SamplingParams
    name = "B"
    folder = model_folders(name)
    ps = PAGE_SIZE[name]
    cfg = EngineConfig(dtype="float32", page_size=ps, max_gpu_num_blocks=None, max_seq_len=128, max_num_seqs=4, timing=True,
                       compiled_model=True)
    llm = LLM(folder, cfg)
    eng = llm.engine
    cap = 4 * (128 // ps)
    rep = eng.memory_report
    assert rep["pages"] == cap == rep["pages_ever_needed"] and rep["pages_that_fit"] > cap
    assert eng.cache.free_pages() == cap
    prompts = [random_tokens(n, 384, 1500 + n) for n in (9, 33, 70)]
    want = _plain_greedy(folder, prompts, 6, [382, 383])
    assert llm.generate(prompts, SamplingParams(temperature=0.0, max_gen_len=6)) == want
    summary = eng.stats.summary()
    assert summary["steps"] >= 6 and summary["tokens"] >= sum(len(p) for p in prompts)
    assert summary["step_ms_mean"] > 0 and summary["peak_pages_used"] >= -(-70 // ps)
    assert {"product", "norm", "attention"} <= set(summary["kernel_ms"]) and all(v > 0 for v in summary["kernel_ms"].values())
    assert not eng._graphs                                           # timed steps run uncaptured
    out = eng.step([StepEntry("x", prompts[2], [69]), StepEntry("y", prompts[0][:1], [])])
    assert out.num_tokens == 71 and out.num_requests == 2
    assert out.pages_used == -(-70 // ps) + 1 and out.pages_used + out.pages_free == cap
    assert out.step_ms > 0 and abs(sum(out.kernel_ms.values()) - out.step_ms) < out.step_ms   # the classes add up to about the step
    eng.finish_all()
    # a fraction of the free memory that leaves room for ten pages only: the pool is what fits, not the cap
    free, _ = torch.cuda.mem_get_info()
    per_page = eng.memory_report["bytes_per_page_all_groups"]
    small = EngineConfig(dtype="float32", page_size=ps, max_gpu_num_blocks=None, max_seq_len=128, max_num_seqs=4,
                         gpu_memory_fraction=((2 << 30) + 10.5 * per_page) / free)
    eng2 = Engine(folder, small)
    assert 8 <= eng2.memory_report["pages"] <= 10 and eng2.cache.free_pages() == eng2.memory_report["pages"]
    with pytest.raises(Exception, match="no memory left"):
        Engine(folder, EngineConfig(dtype="float32", page_size=ps, max_gpu_num_blocks=None, max_seq_len=128, max_num_seqs=4,
                                    gpu_memory_fraction=1e-6))


def test_command_line_prints_statistics(model_folders):
    folder = model_folders("A")
    prompt = random_tokens(7, 256, 700)
    out = subprocess.run([sys.executable, str(ROOT / "cli.py"), "--checkpoints_dir", str(folder), "--dtype", "float32", "--temperature", "0",
                          "--max_gen_len", "5", "--max_seq_len", "64", "--page_size", "4", "--stats", "--prompt_ids"]
                         + [str(t) for t in prompt], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stderr.splitlines() if l.startswith("[stats]")]
    assert len(lines) == 2 and "cache pool" in lines[0] and '"pages"' in lines[0]
    import json
    stats = json.loads(lines[1][len("[stats] "):])
    assert stats["steps"] >= 5 and stats["step_ms_mean"] > 0 and "product" in stats["kernel_ms"]


def test_command_line_with_text_prompts_in_the_chat_form(model_folders, tmp_path):
    """Text prompts: a folder with a small word-level tokenizer that knows the Llama 3 role headers.
    The prompt loop wraps every line in the chat form with the conversation so far (the second
    turn's input holds the first turn and its answer), ``--raw_prompt`` passes lines as they are;
    the tokens generated are those of the same ids given directly."""
    import json
    import shutil
    from tokenizers import Tokenizer, models, pre_tokenizers
    folder = tmp_path / "with_tokenizer"
    shutil.copytree(model_folders("A"), folder)
    words = ["<pad>", "<|begin_of_text|>", "<|eot_id|>", "<|start_header_id|>", "<|end_header_id|>", "user", "assistant", "system",
             "hello", "world", "again"] + [f"w{i}" for i in range(200)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<pad>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.add_special_tokens(["<|begin_of_text|>", "<|eot_id|>", "<|start_header_id|>", "<|end_header_id|>"])
    tok.save(str(folder / "tokenizer.json"))
    (folder / "tokenizer_config.json").write_text(json.dumps(
        {"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<|eot_id|>", "pad_token": "<pad>", "unk_token": "<pad>"}))
    base = [sys.executable, str(ROOT / "cli.py"), "--checkpoints_dir", str(folder), "--dtype", "float32", "--temperature", "0",
            "--max_gen_len", "4", "--max_seq_len", "128", "--max_gpu_num_blocks", "40", "--page_size", "4"]
    from transformers import AutoTokenizer
    hf = AutoTokenizer.from_pretrained(str(folder), use_fast=True)
    chat_ids = hf.encode("<|start_header_id|>user<|end_header_id|>\n\nhello world<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n")
    assert chat_ids[:3] == [3, 5, 4] and 2 in chat_ids                       # header tokens and <|eot_id|> are single tokens
    want_chat = _plain_greedy(model_folders("A"), [chat_ids], 4, [255, 2])[0]
    want_raw = _plain_greedy(model_folders("A"), [hf.encode("hello world")], 4, [255, 2])[0]

    def cut(ids):
        return ids[: next((i for i, t in enumerate(ids) if t in (255, 2)), len(ids))]
    one = subprocess.run(base + ["--prompt", "hello world"], capture_output=True, text=True, timeout=600)
    assert one.returncode == 0, one.stderr[-2000:]
    assert one.stdout.split() == hf.decode(cut(want_chat)).split()
    raw = subprocess.run(base + ["--raw_prompt", "--prompt", "hello world"], capture_output=True, text=True, timeout=600)
    assert raw.returncode == 0, raw.stderr[-2000:]
    assert raw.stdout.split() == hf.decode(cut(want_raw)).split()
    # two turns in the loop: the second answer continues a conversation that holds the first one
    loop = subprocess.run(base, input="hello world\nagain\nexit\n", capture_output=True, text=True, timeout=600)
    assert loop.returncode == 0, loop.stderr[-2000:]
    first_answer = hf.decode(cut(want_chat)).strip()
    second_ids = hf.encode("<|start_header_id|>user<|end_header_id|>\n\nhello world<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n"
                           + first_answer + "<|eot_id|><|start_header_id|>user<|end_header_id|>\n\nagain<|eot_id|>"
                           "<|start_header_id|>assistant<|end_header_id|>\n\n")
    want_second = _plain_greedy(model_folders("A"), [second_ids], 4, [255, 2])[0]
    assert " ".join(hf.decode(cut(want_second)).split()) in " ".join(loop.stdout.split())
