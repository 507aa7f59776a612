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


def _llm(folder, name, pages, overlap, max_seq_len=96, max_num_seqs=4, budget=24):
    from pytriton_llama_b200.engine.llm import LLM
    cfg = EngineConfig(dtype="float32", page_size=PAGE_SIZE[name], max_gpu_num_blocks=pages, max_seq_len=max_seq_len,
                       max_num_seqs=max_num_seqs, max_batched_tokens=budget, overlap_steps=overlap, seed=3)
    return LLM(folder, cfg, device="cpu", ops=TorchOps())


@pytest.mark.parametrize("name", ["A", "B"])
def test_overlapped_steps_generate_the_same_tokens(model_folders, name):
    """Launching the next step before the last one's tokens are read changes nothing in what is
    generated: greedy and sampled, with stop tokens that end requests early, limits known in
    advance, and so few pages that requests are pre-empted and recomputed."""
    from pytriton_llama_b200.sampling.params import SamplingParams
    folder = model_folders(name)
    vocab = TINY[name]["vocab_size"]
    prompts = [random_tokens(n, vocab, 300 + i) for i, n in enumerate([7, 30, 3, 18, 11, 26])]
    ps = PAGE_SIZE[name]
    # greedy first, to find tokens that do occur and use them as stop tokens
    base = _llm(folder, name, 64, overlap=False).generate(prompts, SamplingParams(temperature=0.0, max_gen_len=12))
    stops = sorted({o[5] for o in base} | {base[0][2]})
    settings = [SamplingParams(temperature=0.0, max_gen_len=12, stop_token_ids=stops),
                SamplingParams(temperature=0.9, top_p=0.8, max_gen_len=9, stop_token_ids=stops[:1], logprobs=True),
                SamplingParams(temperature=0.0, max_gen_len=1),
                SamplingParams(temperature=0.0, max_gen_len=None)]           # runs into max_seq_len
    preempted = 0
    for pages in (64, -(-(30 + 12) // ps) + 3):                              # roomy; tight enough to pre-empt
        for sp in settings:
            runs = []
            for overlap in (False, True):
                llm = _llm(folder, name, pages, overlap, max_seq_len=48 if sp.max_gen_len is None else 96)
                reqs = [llm.add_request(p, sp) for p in prompts]
                steps = sum(1 for _ in llm.run())
                runs.append(([list(r.output) for r in reqs], [r.finish_reason for r in reqs],
                             [list(r.logprobs) for r in reqs], sum(r.preemptions for r in reqs)))
                llm.engine.cache.check_invariants()
                assert llm.engine.cache.free_pages() == pages and not llm.scheduler.has_work() and steps > 0
                assert all(-1 not in r.output for r in reqs)
            assert runs[0][:2] == runs[1][:2], (pages, sp)
            for a, b in zip(runs[0][2], runs[1][2]):         # what else is in a batch moves the last bits of a logit
                assert len(a) == len(b) and all(abs(x - y) < 1e-4 for x, y in zip(a, b)), (pages, sp)
            if sp.logprobs:
                assert [len(lp) for lp in runs[1][2]] == [len(o) for o in runs[1][0]]
            preempted += runs[1][3] if pages < 64 else 0
    assert preempted > 0, "the tight cache pre-empted nothing"
    assert any(len(o) < 12 for o in _llm(folder, name, 64, True).generate(prompts, settings[0])), "no stop token ended a request"


def test_partial_rotary_factor_rotates_the_leading_part_of_every_head(tmp_path):
    """config.json's partial_rotary_factor (read by lite_llama/models/RotaryEmbedding.py:43): the
    engine and the plain implementation rotate the first head_dim * factor elements of a head."""
    from conftest import make_model_folder
    from pytriton_llama_b200.weights import write_random_model
    cfg = dict(TINY["B"], partial_rotary_factor=0.5)
    folder = write_random_model(tmp_path / "half", cfg, seed=21, dtype=torch.float32, std=0.08)
    pcfg, w = plain_llama.load_model_folder(folder, dtype=torch.float64)
    assert pcfg["partial_rotary_factor"] == 0.5
    seqs = {f"r{i}": random_tokens(n, 384, 900 + i) for i, n in enumerate([9, 40, 70])}
    ref = {r: plain_llama.forward(pcfg, w, s) for r, s in seqs.items()}
    full = plain_llama.forward(dict(pcfg, partial_rotary_factor=1.0), w, seqs["r2"])
    assert (full - ref["r2"]).abs().max() > 1e-2, "the factor changes nothing in the plain implementation"
    eng = Engine(folder, EngineConfig(dtype="float32", page_size=8, max_gpu_num_blocks=40, max_seq_len=128, max_num_seqs=3),
                 device="cpu", ops=TorchOps())
    got = traces.replay(eng, traces.portions(seqs))
    for r in seqs:
        assert (got[r].double() - ref[r]).abs().max() < FP32_TOL, r


def test_padded_shapes_of_captured_steps(model_folders):
    """The shape a step with prompt portions is padded to before it is captured in a graph: few
    values per dimension, always room for what the step holds, a spare token row whenever single-token
    items are padded, nothing for steps that are too large or want too many rows, and a shape only
    from its second appearance on."""
    from types import SimpleNamespace
    from pytriton_llama_b200.engine.engine import _HostBatch
    from pytriton_llama_b200.ops.cuda import CudaOps
    eng = _engine(model_folders("A"), "A", 16)
    # the work lists are the CUDA operator set's; its planning is host arithmetic and runs here too
    plan = lambda q_lens, starts: CudaOps.plan_step(SimpleNamespace(QUERY_TILE=CudaOps.QUERY_TILE), q_lens, starts)
    eng.ops.WORK_LISTS, eng.ops.plan_step = CudaOps.WORK_LISTS, plan

    def batch(q_lens, wants):
        entries = [StepEntry(f"r{i}", [0] * n, []) for i, n in enumerate(q_lens)]
        return _HostBatch(entries, q_lens, [0] * len(q_lens), [1] * len(q_lens), list(range(len(q_lens))), {}, list(range(wants)),
                          work=plan(q_lens, [0] * len(q_lens)))

    def shape_of(q_lens, wants=1):
        eng._shape_seen.clear()
        assert eng._shape_bucket(batch(q_lens, wants)) == 0          # the first time a shape is only counted
        return eng._shape_bucket(batch(q_lens, wants))

    def shape(t_pad, r_pad, wants, items, tiles):
        return (t_pad, r_pad, wants, (("decode_items", items), ("prefill_tiles", tiles)))

    assert shape_of([300]) == shape(384, 1, 1, 0, 4)                  # 300 tokens -> 384, one pair of tiles per 256 rows
    assert shape_of([30]) == shape(64, 1, 1, 0, 2)
    assert shape_of([30], wants=0) == shape(64, 1, 0, 0, 2)
    assert shape_of([1000, 1, 1, 1], wants=4) == shape(1024, 4, 1, 4, 8)   # 1,003 tokens: 21 spare rows for the fourth, padded item
    assert shape_of([61, 1, 1, 1], wants=4) == shape(128, 4, 1, 4, 2)      # 64 tokens fill 64 rows: the padded item needs one more
    assert shape_of([62, 1, 1], wants=3) == shape(64, 4, 1, 2, 2)          # no item is padded: no spare row needed
    assert shape_of([1025]) == 0 and shape_of([500, 600]) == 0        # more than 1,024 tokens
    assert shape_of([40], wants=2) == 0                               # more wanted rows than padded requests
    eng._shape_captures = eng.GRAPH_MAX_CAPTURES                       # a workload that has captured again and again: no new shapes
    assert shape_of([300]) == 0
    eng._shape_captures = 0
    for q_lens in ([5, 1, 300, 1, 1], [2, 2], [257], [256, 1]):
        b = batch(q_lens, len(q_lens))
        t_pad, r_pad, _, lists = shape_of(q_lens, len(q_lens))
        lists = dict(lists)
        assert t_pad >= b.T and r_pad >= b.R
        assert lists["decode_items"] >= len(b.work["decode_items"]) and lists["prefill_tiles"] >= len(b.work["prefill_tiles"]) // 4
        assert lists["decode_items"] == len(b.work["decode_items"]) or t_pad > b.T
    # an operator set without work lists (the plain one of the tests) pads tokens and requests only
    del eng.ops.WORK_LISTS, eng.ops.plan_step
    eng._shape_seen.clear()
    plain = _HostBatch([StepEntry("r0", [0] * 30, [])], [30], [0], [1], [0], {}, [0])
    assert eng._shape_bucket(plain) == 0 and eng._shape_bucket(plain) == (64, 1, 1, ())


def test_rope_parts_with_equal_parameters_share_their_table():
    """An operator set tells frequency tables apart by address when it works a step's angles out
    once for all layers; layers with the same parameters must therefore hold the same tensor."""
    from pytriton_llama_b200.parts.base import PartSpec, Runtime, build_part
    rt = Runtime(torch.device("cpu"), torch.float32, None)
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64}
    a = build_part("position", PartSpec("rope", {"head_dim": 64, "theta": 1e4, "scaling": dict(scaling)}), rt)
    b = build_part("position", PartSpec("rope", {"head_dim": 64, "theta": 1e4, "scaling": dict(scaling)}), rt)
    c = build_part("position", PartSpec("rope", {"head_dim": 64, "theta": 5e5, "scaling": dict(scaling)}), rt)
    d = build_part("position", PartSpec("rope", {"head_dim": 64, "theta": 1e4, "scaling": None}), rt)
    assert a.inv_freq is b.inv_freq
    assert a.inv_freq is not c.inv_freq and a.inv_freq is not d.inv_freq
    assert not torch.equal(a.inv_freq, d.inv_freq)


def test_a_position_part_without_a_table_rotates_q_and_k_itself(tmp_path):
    """A position encoding that is no rotation of (j, j + rot/2) pairs answers ``rotary_table()``
    with None; the mixer then calls its ``apply`` on the projected q and k before they are stored.
    Interleaved-pair rotary, registered by the test, against a plain float64 statement (the GPU test
    of the same name in test_gpu_parts.py runs it through the kernels)."""
    import test_gpu_parts as toys
    from pytriton_llama_b200.config import LlamaConfig, register_architecture
    from pytriton_llama_b200.models.llama import llama_spec
    from pytriton_llama_b200.parts import PartSpec
    from pytriton_llama_b200.weights import read_folder, write_random_model
    toys._register_toy_interleaved_rotary()
    cfg = dict(TINY["B"], architectures=["ToyInterleavedHostForCausalLM"])

    def spec(c, norm_init="ones"):
        sp = llama_spec(LlamaConfig.from_dict(cfg), norm_init="ones_jitter")
        for layer in sp.layers:
            layer.parts["mixer"].parts["position"] = PartSpec("toy_interleaved_rotary", {"head_dim": LlamaConfig.from_dict(cfg).head_dim})
        return sp

    register_architecture("ToyInterleavedHostForCausalLM", LlamaConfig.from_dict, spec)
    folder = write_random_model(tmp_path / "interleaved", cfg, seed=13, dtype=torch.float32, std=0.08)
    w = {k: v.double() for k, v in read_folder(folder).items()}
    seqs = {f"p{i}": random_tokens(n, 384, 170 + i) for i, n in enumerate([37, 9, 50])}
    ref = {r: toys._plain_interleaved_forward(cfg, w, s) for r, s in seqs.items()}
    eng = Engine(folder, EngineConfig(dtype="float32", page_size=8, max_gpu_num_blocks=24, max_seq_len=128, max_num_seqs=3),
                 device="cpu", ops=TorchOps())
    got = traces.replay(eng, traces.mixed(seqs, live=3))
    for r in seqs:
        assert (got[r].double() - ref[r]).abs().max() < FP32_TOL, r
    # and the plain statement really depends on the pairing: rotate-half gives other logits
    plain = plain_llama.forward(dict(cfg, rope_theta=100.0, rope_scaling=None), w, seqs["p0"])
    assert (plain - ref["p0"]).abs().max() > 1e-2
