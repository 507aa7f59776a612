"""The paged cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice."""
import random

import pytest
import torch

from pytriton_llama_b200.cache.manager import CacheManager, OutOfPages, OutOfSlots, PagePool
from pytriton_llama_b200.parts.base import CacheNeed

FULL = CacheNeed(kind="full", kv_heads=2, head_dim=16)
WINDOW = CacheNeed(kind="window", kv_heads=1, head_dim=32, window=10)
STATE = CacheNeed(kind="none", state_shape=(3, 4), state_dtype=torch.float32)


def manager(entries=None, pages=8, page_size=4, max_requests=4, max_seq_len=64, allocate=True):
    entries = entries or {0: FULL, 1: FULL}
    return CacheManager(entries, page_size, pages, max_requests, max_seq_len, "cpu", torch.float32, allocate=allocate)


def test_pool_take_and_give_back():
    pool = PagePool(4)
    a = pool.take(3)
    assert len(set(a)) == 3 and pool.free_pages == 1
    with pytest.raises(OutOfPages):
        pool.take(2)
    pool.give_back(a[0])
    with pytest.raises(ValueError):
        pool.give_back(a[0])           # freed twice
    assert pool.take(1) == [a[0]]      # the page freed last is used again first
    pool.check()


def test_layers_with_equal_needs_share_a_group_and_pages():
    m = manager({0: FULL, 1: FULL, 2: WINDOW, 3: STATE})
    assert len(m.groups) == 3
    assert m.groups[m.entry_group[0]].entries == [0, 1]
    assert m.groups[m.entry_group[0]].kv[1].shape == (8, 2, 2, 4, 16)
    assert m.groups[m.entry_group[2]].kv[2].shape == (8, 2, 1, 4, 32)
    assert m.groups[m.entry_group[3]].pool is None
    assert m.groups[m.entry_group[3]].state[3].shape == (4, 3, 4)


def test_append_gives_slots_page_by_page():
    m = manager()
    m.admit("a")
    slots = m.append("a", 6)[0]
    t = m.block_table("a", 0)
    assert len(t) == 2
    assert slots == [t[0] * 4 + i for i in range(4)] + [t[1] * 4, t[1] * 4 + 1]
    slots = m.append("a", 3)[0]                      # fills the second page, opens a third
    t = m.block_table("a", 0)
    assert slots == [t[1] * 4 + 2, t[1] * 4 + 3, t[2] * 4]
    assert m.tokens_of("a") == 9 and m.free_pages() == 5
    m.check_invariants()


def test_out_of_pages_takes_nothing():
    m = manager(pages=3)
    m.admit("a")
    m.append("a", 8)
    m.admit("b")
    assert not m.can_append([("b", 5)])
    assert m.can_append([("b", 4)])
    with pytest.raises(OutOfPages):
        m.append("b", 5)
    assert m.tokens_of("b") == 0 and m.free_pages() == 1
    m.check_invariants()
    m.release("a")
    assert m.free_pages() == 3
    m.append("b", 12)
    m.check_invariants()


def test_slots_run_out_and_come_back():
    m = manager(max_requests=2)
    s0, s1 = m.admit("a"), m.admit("b")
    assert s0 != s1
    with pytest.raises(OutOfSlots):
        m.admit("c")
    with pytest.raises(ValueError):
        m.admit("a")
    m.release("a")
    assert m.admit("c") == s0
    m.check_invariants()


def test_state_is_zeroed_at_admission():
    m = manager({0: STATE}, max_requests=2)
    st = m.groups[0].state[0]
    slot = m.admit("a")
    st[slot] += 5
    m.release("a")
    assert m.admit("b") == slot
    assert st[slot].abs().sum() == 0


def test_window_group_gives_pages_back_once_the_window_has_passed():
    m = manager({0: WINDOW}, pages=6, page_size=4, max_seq_len=200)
    m.admit("a")
    held = []
    for step in range(40):                           # 40 tokens one by one, window 10, pages of 4
        m.append("a", 1)
        n = m.tokens_of("a")
        t = m.block_table("a", 0)
        first_key = max(0, (n - 1) - 10 + 1)         # oldest key the newest token sees
        for b, p in enumerate(t):
            if b * 4 + 3 >= first_key and b * 4 < n:
                assert p >= 0, f"block {b} is still visible at {n} tokens but was given back"
        held.append(sum(1 for p in t if p >= 0))
        m.check_invariants()
    assert max(held) <= 4                            # ceil((10 + 3) / 4) + 1 pages at most, never 10
    assert m.free_pages() == 6 - held[-1]
    m.release("a")
    assert m.free_pages() == 6


def test_window_portion_keeps_what_its_first_token_sees():
    m = manager({0: WINDOW}, pages=10, page_size=4, max_seq_len=200)
    m.admit("a")
    m.append("a", 21)
    m.append("a", 7)                                  # queries at 21..27; the one at 21 sees keys 12..21
    t = m.block_table("a", 0)
    assert all(p >= 0 for p in t[3:]) and all(p < 0 for p in t[:3])
    m.check_invariants()


def test_sequence_limit():
    m = manager(max_seq_len=10)
    m.admit("a")
    m.append("a", 10)
    with pytest.raises(ValueError):
        m.append("a", 1)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_books(seed):
    rng = random.Random(seed)
    m = manager({0: FULL, 1: FULL, 2: WINDOW, 3: STATE}, pages=12, page_size=4, max_requests=5, max_seq_len=40)
    live = {}
    next_id = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.free_slots():
            rid = f"r{next_id}"
            next_id += 1
            m.admit(rid)
            live[rid] = 0
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7])
            if live[rid] + n > 40:
                continue
            ok = m.can_append([(rid, n)])
            before = [m.free_pages(g) for g in range(len(m.groups))]
            try:
                slots = m.append(rid, n)
                assert ok
                live[rid] += n
                for g, sl in slots.items():
                    assert len(sl) == n and len(set(sl)) == n
            except OutOfPages:
                assert not ok
                assert before == [m.free_pages(g) for g in range(len(m.groups))]
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        assert {r: m.tokens_of(r) for r in live} == live
    # no two live requests ever share a slot of the cache
    seen = set()
    for rid in live:
        for g in (0, 1):
            for p in m.block_table(rid, g):
                if p >= 0:
                    assert (g, p) not in seen
                    seen.add((g, p))
    m.release_all()
    assert all(m.free_pages(g) == 12 for g in (0, 1)) and m.free_slots() == 5
