"""The scheduler's decisions (no GPU): admission, portions under a token budget, decoding,
finishing, and what happens when pages run out."""
import torch

from pytriton_llama_b200.cache.manager import CacheManager
from pytriton_llama_b200.engine.scheduler import Scheduler
from pytriton_llama_b200.parts.base import CacheNeed
from pytriton_llama_b200.sampling import SamplingParams

FULL = CacheNeed(kind="full", kv_heads=1, head_dim=16)


def make(pages=16, page_size=4, max_num_seqs=4, budget=16, max_seq_len=64, eos=(99,)):
    cache = CacheManager({0: FULL}, page_size, pages, max_num_seqs, max_seq_len, "cpu", torch.float32, allocate=False)
    return cache, Scheduler(cache, max_num_seqs, budget, max_seq_len, eos_token_ids=eos)


def run_plan(cache, sched, plan, token=1):
    """What the engine does with a plan: take the pages, then report one sampled token per finished portion."""
    for p in plan.portions:
        if not cache.has(p.request.id):
            cache.admit(p.request.id)
        cache.append(p.request.id, p.length)
    cache.check_invariants()
    sampled = {p.request.id: (token(p.request) if callable(token) else token) for p in plan.portions if p.sample}
    return sched.update(plan, sampled)


def test_prompts_are_cut_under_the_token_budget():
    cache, s = make(budget=16)
    a = s.add("a", list(range(40)), SamplingParams(max_gen_len=3))
    b = s.add("b", list(range(5)), SamplingParams(max_gen_len=3))
    plan = s.schedule()
    assert [(p.request.id, p.start, p.length, p.sample) for p in plan.portions] == [("a", 0, 16, False)]
    run_plan(cache, s, plan)
    plan = s.schedule()
    assert [(p.request.id, p.start, p.length) for p in plan.portions] == [("a", 16, 16)]
    run_plan(cache, s, plan)
    plan = s.schedule()      # a's last 8 prompt tokens, b's whole prompt beside them
    assert [(p.request.id, p.start, p.length, p.sample) for p in plan.portions] == [("a", 32, 8, True), ("b", 0, 5, True)]
    run_plan(cache, s, plan)
    assert a.output == [1] and b.output == [1]
    plan = s.schedule()      # both decode: one token each
    assert [(p.request.id, p.start, p.length, p.sample) for p in plan.portions] == [("a", 40, 1, True), ("b", 5, 1, True)]


def test_decode_tokens_come_before_new_prompts_and_share_the_step():
    cache, s = make(budget=8)
    s.add("a", [1, 2, 3], SamplingParams(max_gen_len=10))
    run_plan(cache, s, s.schedule())
    s.add("b", list(range(20)), SamplingParams(max_gen_len=2))
    plan = s.schedule()
    assert [(p.request.id, p.length) for p in plan.portions] == [("a", 1), ("b", 7)]
    assert plan.num_tokens == 8


def test_finishing_by_stop_token_length_and_sequence_limit():
    cache, s = make(max_seq_len=8)
    a = s.add("a", [1, 2], SamplingParams(max_gen_len=2))
    b = s.add("b", [1, 2], SamplingParams(max_gen_len=50))
    c = s.add("c", [1, 2, 3], SamplingParams(max_gen_len=50, stop_token_ids=[7]))
    tokens = {"a": iter([5, 5, 5]), "b": iter([5, 5, 99]), "c": iter([5, 7])}
    done = []
    while s.has_work():
        plan = s.schedule()
        done += run_plan(cache, s, plan, token=lambda r: next(tokens[r.id]))
    assert (a.finish_reason, a.output) == ("length", [5, 5])
    assert (b.finish_reason, b.output) == ("stop", [5, 5, 99])         # the engine's end-of-sequence id
    assert (c.finish_reason, c.output) == ("stop", [5, 7])             # the request's own stop id
    assert cache.free_pages() == 16 and cache.free_slots() == 4        # everything given back
    d = s.add("d", [1, 2, 3], SamplingParams(max_gen_len=50))
    while s.has_work():
        run_plan(cache, s, s.schedule(), token=5)
    assert d.finish_reason == "max_seq_len" and len(d.prompt) + len(d.output) == 8


def test_bad_prompts_finish_at_once():
    cache, s = make(max_seq_len=8)
    assert s.add("a", []).finish_reason == "empty_prompt"
    assert s.add("b", list(range(8))).finish_reason == "prompt_too_long"
    assert not s.has_work()


def test_no_more_live_requests_than_slots():
    cache, s = make(max_num_seqs=2, budget=64)
    for i in range(4):
        s.add(i, [1, 2, 3], SamplingParams(max_gen_len=2))
    plan = s.schedule()
    assert [p.request.id for p in plan.portions] == [0, 1]
    run_plan(cache, s, plan)
    run_plan(cache, s, s.schedule())          # 0 and 1 reach their length and leave
    plan = s.schedule()
    assert [p.request.id for p in plan.portions] == [2, 3]


def test_new_prompts_wait_while_pages_are_short():
    cache, s = make(pages=4, page_size=4, budget=64)      # 16 tokens of cache
    s.add("a", list(range(10)), SamplingParams(max_gen_len=4))
    s.add("b", list(range(10)), SamplingParams(max_gen_len=4))
    plan = s.schedule()
    assert [p.request.id for p in plan.portions] == ["a"]  # b's 10 tokens need 3 pages, 1 is free
    run_plan(cache, s, plan)
    while any(r.id == "a" for r in s.running):
        plan = s.schedule()
        assert [p.request.id for p in plan.portions] == ["a"]
        run_plan(cache, s, plan)
    plan = s.schedule()
    assert [(p.request.id, p.length) for p in plan.portions] == [("b", 10)]   # in the pages a gave back


def test_running_out_of_pages_preempts_the_youngest_request_which_recomputes_later():
    cache, s = make(pages=6, page_size=4, budget=64)      # 24 tokens of cache
    a = s.add("a", list(range(11)), SamplingParams(max_gen_len=8))
    b = s.add("b", list(range(11)), SamplingParams(max_gen_len=8))
    plan = s.schedule()
    assert [p.request.id for p in plan.portions] == ["a", "b"]      # 3 + 3 pages
    run_plan(cache, s, plan, token=5)
    plan = s.schedule()                                             # both decode into their third page
    assert not plan.preempted
    run_plan(cache, s, plan, token=5)
    plan = s.schedule()                                             # token 13 of each needs a fourth page: none left
    assert [r.id for r in plan.preempted] == ["b"]
    assert [p.request.id for p in plan.portions] == ["a"]
    assert b.status == "waiting" and b.computed == 0 and b.output == [5, 5] and b.preemptions == 1
    assert not cache.has("b")
    run_plan(cache, s, plan, token=5)
    outputs = {}
    while s.has_work():
        plan = s.schedule()
        for p in plan.portions:
            if p.request is b and p.start == 0:
                outputs["recompute"] = p.length                     # prompt and its generated tokens together
        run_plan(cache, s, plan, token=5)
    assert outputs["recompute"] == 11 + len([5, 5])
    assert a.finish_reason == b.finish_reason == "length" and len(a.output) == len(b.output) == 8
    assert cache.free_pages() == 6
    cache.check_invariants()


def test_a_request_that_can_never_fit_ends_instead_of_hanging():
    cache, s = make(pages=2, page_size=4, budget=64)      # 8 tokens of cache
    big = s.add("big", list(range(20)), SamplingParams(max_gen_len=4))
    ok = s.add("ok", [1, 2, 3], SamplingParams(max_gen_len=2))
    steps = 0
    while s.has_work():
        plan = s.schedule()
        run_plan(cache, s, plan, token=5)
        steps += 1
        assert steps < 50
    assert big.finish_reason == "cache_too_small" and big.output == []
    assert ok.finish_reason == "length"
    # one that fits at first but outgrows the whole cache while decoding
    cache, s = make(pages=2, page_size=4, budget=64)
    grow = s.add("grow", list(range(6)), SamplingParams(max_gen_len=30))
    steps = 0
    while s.has_work():
        run_plan(cache, s, s.schedule(), token=5)
        steps += 1
        assert steps < 50
    assert grow.finish_reason == "cache_too_small" and len(grow.output) == 3   # 6 + 2 fill the cache; the third token found no page
    assert cache.free_pages() == 2


def test_uniform_numbers_depend_only_on_their_counters():
    from pytriton_llama_b200.sampling import uniform
    assert uniform(1, 2, 3) == uniform(1, 2, 3)
    vals = {uniform(s, r, i) for s in range(3) for r in range(5) for i in range(20)}
    assert len(vals) == 300 and all(0 <= v < 1 for v in vals)
    assert abs(sum(vals) / 300 - 0.5) < 0.06
