"""Paged cache manager: pages with a block table per request, one pool per group of cache entries
with the same need, and slots for per-request state of fixed size.

lite_llama's manager hands out single token slots from a device-side use-count array and
reserves a batch's whole life up front (lite_llama/executor/mem_manager.py:134-220,
lite_llama/generate.py:111-127); its request table gives each request a slot index
(lite_llama/executor/req_tokens_table.py:15-29).  Here the unit is a page of ``page_size``
tokens, pages are taken when a step needs them and given back when a request ends or, in a
windowed group, when the window has passed them; the bookkeeping lives on the host.

Cache entries (one per run of a layer that stores keys and values) with equal needs form a
group.  A page id is valid in every entry of its group: entry e keeps its share of page p in
``kv[e][p]`` of shape [2 (k, v), kv_heads, page_size, head_dim].
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Tuple

import numpy as np
import torch

from ..parts.base import CacheNeed


class OutOfPages(RuntimeError):
    """A pool has too few free pages for what was asked."""


class OutOfSlots(RuntimeError):
    """Every per-request slot is taken."""


class PagePool:
    """Free list and use counts of the pages of one group (host side)."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # a stack: the page freed last is used first
        self._count = [0] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free of {self.num_pages}")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            assert self._count[p] == 0, f"page {p} handed out while in use"
            self._count[p] = 1
        return pages

    def share(self, page: int) -> None:
        if self._count[page] <= 0:
            raise ValueError(f"page {page} is not in use")
        self._count[page] += 1

    def give_back(self, page: int) -> None:
        if not 0 <= page < self.num_pages or self._count[page] <= 0:
            raise ValueError(f"page {page} is given back but not in use")
        self._count[page] -= 1
        if self._count[page] == 0:
            self._free.append(page)

    def check(self) -> None:
        free = set(self._free)
        assert len(free) == len(self._free), "a page is in the free list twice"
        for p in range(self.num_pages):
            assert (self._count[p] == 0) == (p in free), f"page {p}: count {self._count[p]}, free={p in free}"


@dataclass
class CacheGroup:
    need: CacheNeed
    entries: List[int]
    page_size: int
    pool: Optional[PagePool]                       # None for groups that keep no keys/values
    kv: Dict[int, torch.Tensor] = field(default_factory=dict)
    state: Dict[int, torch.Tensor] = field(default_factory=dict)

    @property
    def paged(self) -> bool:
        return self.pool is not None

    def page_bytes(self, element_size: int) -> int:
        n = self.need
        return 2 * n.kv_heads * n.head_dim * self.page_size * element_size * len(self.entries)


class _Table:
    """Block table of one request in one group: page of each block (-1: given back), kept in a
    numpy array so that a step can copy it into its batch without a Python loop."""
    __slots__ = ("pages", "n")

    def __init__(self, capacity: int):
        self.pages = np.full(capacity, -1, dtype=np.int32)
        self.n = 0

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, i):
        if isinstance(i, slice):
            return self.pages[:self.n][i].tolist()
        return int(self.pages[i])

    def __setitem__(self, i: int, v: int) -> None:
        self.pages[i] = v

    def __iter__(self):
        return iter(self.pages[:self.n].tolist())

    def extend(self, pages: List[int]) -> None:
        self.pages[self.n:self.n + len(pages)] = pages
        self.n += len(pages)

    def array(self) -> np.ndarray:
        return self.pages[:self.n]

    def held_below(self, block: int) -> int:
        return int((self.pages[:min(block, self.n)] >= 0).sum()) if block > 0 else 0


@dataclass
class _Request:
    slot: int
    tokens: int = 0
    tables: Dict[int, _Table] = field(default_factory=dict)   # group -> block table


class CacheManager:
    def __init__(self, entries: Dict[int, CacheNeed], page_size: int, num_pages: int, max_requests: int,
                 max_seq_len: int, device, dtype: torch.dtype, allocate: bool = True):
        self.page_size = page_size
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self.max_blocks = -(-max_seq_len // page_size)
        self.device = torch.device(device)
        self.dtype = dtype
        self.groups: List[CacheGroup] = []
        self.entry_group: Dict[int, int] = {}
        by_key: Dict[Tuple, int] = {}
        for e in sorted(entries):
            need = entries[e]
            key = need.group_key()
            if key not in by_key:
                by_key[key] = len(self.groups)
                pool = PagePool(num_pages) if need.kind in ("full", "window") else None
                self.groups.append(CacheGroup(need, [], page_size, pool))
            g = by_key[key]
            self.groups[g].entries.append(e)
            self.entry_group[e] = g
        if allocate:
            for grp in self.groups:
                n = grp.need
                for e in grp.entries:
                    if grp.paged:
                        grp.kv[e] = torch.zeros((num_pages, 2, n.kv_heads, page_size, n.head_dim),
                                                dtype=dtype, device=self.device)
                    if n.state_shape is not None:
                        grp.state[e] = torch.zeros((max_requests, *n.state_shape),
                                                   dtype=n.state_dtype or torch.float32, device=self.device)
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}

    # ------------------------------------------------------------------ queries
    def has(self, req: Hashable) -> bool:
        return req in self._requests

    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    def tokens_of(self, req: Hashable) -> int:
        return self._requests[req].tokens

    def slot_of(self, req: Hashable) -> int:
        return self._requests[req].slot

    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self, group: int = 0) -> int:
        pool = self.groups[group].pool
        return pool.free_pages if pool else 0

    def block_table(self, req: Hashable, group: int) -> List[int]:
        t = self._requests[req].tables.get(group)
        return [] if t is None else list(t)

    def block_table_array(self, req: Hashable, group: int) -> np.ndarray:
        """The same as an int32 array (a view: copy it before the next change of the request)."""
        return self._requests[req].tables[group].array()

    def _first_needed_block(self, grp: CacheGroup, next_pos: int) -> int:
        """Blocks below this index hold no key that a query at ``next_pos`` or later can see."""
        if grp.need.kind != "window":
            return 0
        first_key = max(0, next_pos - grp.need.window + 1)
        return first_key // self.page_size

    def pages_needed(self, req: Optional[Hashable], new_tokens: int, have_tokens: Optional[int] = None) -> Dict[int, int]:
        """Group -> pages that appending ``new_tokens`` would take, net of those the append gives back first."""
        if req is not None and req in self._requests:
            r = self._requests[req]
            have = r.tokens
        else:
            r = None
            have = have_tokens or 0
        out = {}
        total_blocks = -(-(have + new_tokens) // self.page_size)
        for gi, grp in enumerate(self.groups):
            if not grp.paged:
                continue
            held = len(r.tables[gi]) if r else -(-have // self.page_size)
            need = total_blocks - held
            if r is not None and grp.need.kind == "window":
                need -= r.tables[gi].held_below(self._first_needed_block(grp, have))
            out[gi] = need
        return out

    def can_append(self, asks: List[Tuple[Optional[Hashable], int]]) -> bool:
        """True if all ``(request, new_tokens)`` asks fit at once (a request None counts as new)."""
        total: Dict[int, int] = {}
        new_requests = 0
        for req, n in asks:
            if req is None or req not in self._requests:
                new_requests += 1
            for g, k in self.pages_needed(req, n).items():
                total[g] = total.get(g, 0) + k
        if new_requests > len(self._free_slots):
            return False
        return all(k <= self.groups[g].pool.free_pages for g, k in total.items())

    # ------------------------------------------------------------------ changes
    def admit(self, req: Hashable) -> int:
        if req in self._requests:
            raise ValueError(f"request {req!r} is already live")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self._requests[req] = _Request(slot=slot, tables={g: _Table(self.max_blocks) for g, grp in enumerate(self.groups) if grp.paged})
        for grp in self.groups:
            for st in grp.state.values():
                st[slot].zero_()
        return slot

    def append(self, req: Hashable, new_tokens: int) -> Dict[int, List[int]]:
        """Makes room for ``new_tokens`` more tokens of ``req``; returns group -> flat slot
        (page * page_size + offset) of each new token.  Takes no page if any group is short."""
        r = self._requests[req]
        if new_tokens <= 0:
            raise ValueError("append needs at least one token")
        if r.tokens + new_tokens > self.max_seq_len:
            raise ValueError(f"request {req!r} would hold {r.tokens + new_tokens} tokens, the limit is {self.max_seq_len}")
        needs = self.pages_needed(req, new_tokens)
        for g, k in needs.items():
            if k > self.groups[g].pool.free_pages:
                raise OutOfPages(f"group {g}: {k} pages wanted, {self.groups[g].pool.free_pages} free")
        ps = self.page_size
        out: Dict[int, List[int]] = {}
        for gi, grp in enumerate(self.groups):
            if not grp.paged:
                continue
            table = r.tables[gi]
            first = self._first_needed_block(grp, r.tokens)
            for b in range(min(first, len(table))):
                if table[b] >= 0:
                    grp.pool.give_back(table[b])
                    table[b] = -1
            total_blocks = -(-(r.tokens + new_tokens) // ps)
            if total_blocks > len(table):
                table.extend(grp.pool.take(total_blocks - len(table)))
            if new_tokens == 1:
                p = r.tokens
                out[gi] = [table[p // ps] * ps + p % ps]
            else:
                pos = np.arange(r.tokens, r.tokens + new_tokens)
                out[gi] = (table.pages[pos // ps].astype(np.int64) * ps + pos % ps).tolist()
        r.tokens += new_tokens
        return out

    def release(self, req: Hashable) -> None:
        r = self._requests.pop(req)
        for gi, table in r.tables.items():
            pool = self.groups[gi].pool
            for p in table:
                if p >= 0:
                    pool.give_back(p)
        self._free_slots.append(r.slot)

    def release_all(self) -> None:
        for req in list(self._requests):
            self.release(req)

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held."""
        for gi, grp in enumerate(self.groups):
            if not grp.paged:
                continue
            grp.pool.check()
            held: Dict[int, Hashable] = {}
            for req, r in self._requests.items():
                for p in r.tables[gi]:
                    if p >= 0:
                        assert p not in held, f"page {p} of group {gi} is held by {held[p]!r} and {req!r}"
                        held[p] = req
            assert len(held) == grp.pool.used_pages, (
                f"group {gi}: {grp.pool.used_pages} pages in use but requests hold {len(held)}")
        slots = [r.slot for r in self._requests.values()]
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert len(slots) + len(self._free_slots) == self.max_requests, "a state slot was lost"
        assert not set(slots) & set(self._free_slots), "a state slot is both free and held"
