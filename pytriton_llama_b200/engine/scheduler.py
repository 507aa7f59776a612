"""Continuous batching above the step function.

lite_llama has no scheduler: a list of prompts is one static batch, padded to the longest
prompt, with the cache for its whole life reserved up front and every request stepping until
the last one ends (lite_llama/generate.py:108-149).  Here requests wait in a queue, are admitted
while slots and pages last, have their prompts cut into portions under a token budget, decode one
token per step beside other requests' portions, and free their pages the moment they finish.

When pages run out for a request that is already running, the request admitted last is
pre-empted: its pages are given back, it returns to the front of the queue and later recomputes
its prompt together with the tokens it had generated.  A request that could not fit even into an
empty cache is finished with reason "cache_too_small" instead of waiting for ever.

A step's outcome is recorded in two halves so that the next step can be planned and launched
while the first one's tokens are still on the device: ``advance`` (right after the launch) counts
the tokens as computed and puts a placeholder where the sampled token will go; ``resolve`` (once
the token has been read) fills it in and ends the request if it was a stop token.  A request that
is known to end with the token in flight (length limits) is set aside and not planned again; one
that ends by a stop token may have run one more step by then, whose token is dropped.
``update`` does both at once.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional

from ..sampling.params import SamplingParams

WAITING, RUNNING, DRAINING, FINISHED = "waiting", "running", "draining", "finished"
PENDING = -1     # stands in ``Request.output`` for a token that was sampled but not read yet


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    number: int = 0                    # arrival number; also feeds the sampling counters
    output: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)   # of the generated tokens, when asked for
    computed: int = 0                  # tokens of prompt + output that are in the cache
    status: str = WAITING
    finish_reason: Optional[str] = None
    preemptions: int = 0

    @property
    def all_tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed

    def tokens(self, start: int, length: int) -> List[int]:
        """``all_tokens[start:start + length]`` without joining the two lists."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n:start - n + length]
        if start + length <= n:
            return self.prompt[start:start + length]
        return self.prompt[start:] + self.output[:start + length - n]


@dataclass
class Portion:
    request: Request
    start: int            # index into all_tokens
    length: int
    sample: bool          # True when the portion ends at the request's last token
    out_index: int = -1   # where in ``request.output`` the sampled token goes (set by ``advance``)


@dataclass
class StepPlan:
    portions: List[Portion] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    finished: List[Request] = field(default_factory=list)   # ended by the scheduler itself (could never fit)

    @property
    def num_tokens(self) -> int:
        return sum(p.length for p in self.portions)


class Scheduler:
    """Decides what each step runs.  ``cache`` is the engine's CacheManager (only its host-side
    bookkeeping is used); pages are actually taken when the engine runs the plan."""

    def __init__(self, cache, max_num_seqs: int, max_batched_tokens: int, max_seq_len: int,
                 eos_token_ids=(), max_portion: Optional[int] = None):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_batched_tokens = max_batched_tokens
        self.max_seq_len = max_seq_len
        self.max_portion = max_portion or max_batched_tokens
        self.eos_token_ids = set(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []      # in admission order
        self.draining: List[Request] = []     # their last token is in flight
        self._counter = 0

    # ------------------------------------------------------------------ intake
    def add(self, request_id: Hashable, prompt: List[int], params: Optional[SamplingParams] = None) -> Request:
        params = params or SamplingParams()
        req = Request(request_id, list(prompt), params, number=self._counter)
        self._counter += 1
        if not req.prompt:
            req.status, req.finish_reason = FINISHED, "empty_prompt"
        elif len(req.prompt) >= self.max_seq_len:
            req.status, req.finish_reason = FINISHED, "prompt_too_long"
        else:
            self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self.draining)

    # ------------------------------------------------------------------ planning
    def _needs(self, req: Request, n: int):
        """(pages per group, slots) that ``n`` more tokens of ``req`` take."""
        live = self.cache.has(req.id)
        return self.cache.pages_needed(req.id if live else None, n), 0 if live else 1

    def _fits(self, needs, slots, reserved, reserved_slots) -> bool:
        if slots + reserved_slots > self.cache.free_slots():
            return False
        return all(k + reserved.get(g, 0) <= self.cache.free_pages(g) for g, k in needs.items())

    def _fits_empty_cache(self, req: Request, n_tokens: int) -> bool:
        blocks = -(-n_tokens // self.cache.page_size)
        for grp in self.cache.groups:
            if grp.paged and grp.need.kind == "full" and blocks > grp.pool.num_pages:
                return False
        return True

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self.running.remove(req)
        if self.cache.has(req.id):
            self.cache.release(req.id)
        req.computed = 0
        req.status = WAITING
        req.preemptions += 1
        self.waiting.appendleft(req)
        plan.preempted.append(req)

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_batched_tokens
        reserved: Dict[int, int] = {}      # pages per group promised to portions accepted so far
        reserved_slots = 0
        accepted: Dict[Hashable, tuple] = {}   # request id -> (needs, slots) it reserved

        def accept(req, n, needs, slots):
            nonlocal budget, reserved_slots
            plan.portions.append(Portion(req, req.computed, n, sample=(n == req.pending)))
            for g, k in needs.items():
                reserved[g] = reserved.get(g, 0) + k
            reserved_slots += slots
            accepted[req.id] = (needs, slots)
            budget -= n

        # 1. running requests, oldest first: one token when decoding, else the next prompt portion
        for req in list(self.running):
            if req not in self.running:
                continue   # pre-empted while serving an older request
            if budget <= 0:
                break
            n = min(req.pending, budget, self.max_portion)
            needs, slots = self._needs(req, n)
            while not self._fits(needs, slots, reserved, reserved_slots):
                victim = self.running[-1]
                if victim is req:
                    # nothing younger to evict: shrink the portion, else give up this request
                    if n > 1:
                        n = max(1, n // 2)
                        needs, slots = self._needs(req, n)
                        continue
                    if self.draining:
                        pass       # pages come back as soon as the tokens in flight have been read: wait a step
                    elif len(self.running) == 1 and not accepted:
                        self.running.remove(req)
                        self.cache.release(req.id)
                        req.status, req.finish_reason = FINISHED, "cache_too_small"
                        plan.finished.append(req)
                    else:
                        self._preempt(req, plan)
                    n = 0
                    break
                # a younger request gives way (it has nothing planned yet: older ones come first)
                self._preempt(victim, plan)
            if n <= 0:
                continue
            accept(req, n, needs, slots)
        # 2. admissions, first come first served, not in a step that had to pre-empt
        while self.waiting and not plan.preempted and budget > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            total = len(req.prompt) + len(req.output)
            if not self._fits_empty_cache(req, total + 1):
                self.waiting.popleft()
                req.status, req.finish_reason = FINISHED, "cache_too_small"
                plan.finished.append(req)
                continue
            n = min(req.pending, budget, self.max_portion)
            needs, slots = self._needs(req, n)
            if not self._fits(needs, slots, reserved, reserved_slots):
                break
            self.waiting.popleft()
            req.status = RUNNING
            self.running.append(req)
            accept(req, n, needs, slots)
        return plan

    # ------------------------------------------------------------------ after the step
    def advance(self, plan: StepPlan) -> None:
        """The plan has been launched: its tokens count as computed, and every portion with
        ``sample`` set gets a placeholder for its token.  Requests that end with that token for a
        reason known now (``max_gen_len``, ``max_seq_len``) are not planned again."""
        for p in plan.portions:
            req = p.request
            req.computed += p.length
            if not p.sample:
                continue
            p.out_index = len(req.output)
            req.output.append(PENDING)
            limit = req.params.max_gen_len
            if limit is not None and len(req.output) >= limit:
                req.finish_reason = "length"
            elif len(req.prompt) + len(req.output) >= self.max_seq_len:
                req.finish_reason = "max_seq_len"
            if req.finish_reason:
                req.status = DRAINING
                self.running.remove(req)
                self.draining.append(req)

    def resolve(self, plan: StepPlan, sampled: Dict[Hashable, int],
                logprobs: Optional[Dict[Hashable, Optional[float]]] = None):
        """The plan's tokens have been read: ``sampled`` has the new token of every portion with
        ``sample`` set.  Returns (request id -> token for the tokens that count, requests that
        finished); the pages of finished requests are given back here."""
        accepted: Dict[Hashable, int] = {}
        done: List[Request] = []
        for p in plan.portions:
            req = p.request
            if not p.sample or req.status == FINISHED:
                continue            # a request that a stop token ended one step earlier: the extra token is dropped
            tok = int(sampled[req.id])
            req.output[p.out_index] = tok
            accepted[req.id] = tok
            if logprobs is not None and logprobs.get(req.id) is not None:
                req.logprobs.append(float(logprobs[req.id]))
            if tok in self.eos_token_ids or tok in req.params.stop_token_ids:
                req.finish_reason = "stop"
                del req.output[p.out_index + 1:]
            elif not (req.status == DRAINING and p.out_index == len(req.output) - 1):
                continue
            if req.status == DRAINING:
                self.draining.remove(req)
            elif req.status == RUNNING:
                self.running.remove(req)
            else:
                self.waiting.remove(req)        # pre-empted while its token was in flight
            req.status = FINISHED
            if self.cache.has(req.id):
                self.cache.release(req.id)
            done.append(req)
        return accepted, done

    def update(self, plan: StepPlan, sampled: Dict[Hashable, int],
               logprobs: Optional[Dict[Hashable, Optional[float]]] = None) -> List[Request]:
        """``advance`` and ``resolve`` in one go, for callers that read the tokens before they plan
        the next step.  Returns the requests that finished."""
        self.advance(plan)
        return self.resolve(plan, sampled, logprobs)[1]
