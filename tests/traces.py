"""Builds replay traces (the JSON steps that ``bin/trace_run`` reads) and replays them in-process.

A trace is a list of steps ``{"step": i, "entries": [{"id", "tokens", "want"}], "end": [...]}``.
The four families cut the same token lists differently; logits at a position must not depend on
the cut beyond rounding.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch


def whole(seqs: Dict[str, List[int]]):
    """Each request alone and whole: one step, every position wanted."""
    steps = []
    for i, (rid, toks) in enumerate(seqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def prefill_then_decode(seqs: Dict[str, List[int]], tail: int = 32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in seqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(seqs: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 5, 3, 2, 16, 2, 9, 4, 2, 31)):
    """Each request alone in portions of changing size, down to two tokens."""
    steps = []
    k = 0
    for rid, toks in seqs.items():
        p = 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}],
                          "end": [rid] if p + n == len(toks) else []})
            p += n
    return steps


def mixed(seqs: Dict[str, List[int]], live: int = 4, sizes: Sequence[int] = (5, 2, 11, 3, 2, 8), decode_tail: int = 6,
          skip_every: int = 5):
    """Up to ``live`` requests at a time: prompt portions of some beside single decoded tokens of
    others; a request is now and then left out of a step; finished requests end and the next ones
    start in the pages they gave back."""
    order = list(seqs)
    pos = {r: 0 for r in order}
    waiting = list(order)
    running: List[str] = []
    steps = []
    k = 0
    while waiting or running:
        while waiting and len(running) < live:
            running.append(waiting.pop(0))
        entries, ended = [], []
        for j, rid in enumerate(list(running)):
            toks = seqs[rid]
            if len(running) > 1 and (len(steps) + j) % skip_every == skip_every - 1:
                continue   # left out of this step, goes on later
            left = len(toks) - pos[rid]
            if left <= decode_tail:
                n = 1
            else:
                n = min(sizes[k % len(sizes)], left - decode_tail)
                k += 1
            entries.append({"id": rid, "tokens": toks[pos[rid]:pos[rid] + n], "want": list(range(n))})
            pos[rid] += n
            if pos[rid] == len(toks):
                ended.append(rid)
                running.remove(rid)
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def random_trace(seqs: Dict[str, List[int]], rng, live: int = 4):
    """A trace drawn from ``rng`` (a ``random.Random``): requests start in random order while others
    run, a step gives a request one token, a few, or up to 140, sometimes leaves it out, and wants
    every place, a random subset of the places, or none."""
    order = list(seqs)
    rng.shuffle(order)
    pos = {r: 0 for r in order}
    waiting, running, steps = list(order), [], []
    while waiting or running:
        while waiting and len(running) < live and (not running or rng.random() < 0.7):
            running.append(waiting.pop(0))
        entries, ended = [], []
        for rid in list(running):
            if len(running) > 1 and rng.random() < 0.2:
                continue
            left = len(seqs[rid]) - pos[rid]
            kind = rng.random()
            n = 1 if kind < 0.45 else rng.randint(2, 12) if kind < 0.8 else rng.randint(13, 140)
            n = min(n, left)
            want = sorted(rng.sample(range(n), rng.randint(0, n))) if rng.random() < 0.3 else list(range(n))
            entries.append({"id": rid, "tokens": seqs[rid][pos[rid]:pos[rid] + n], "want": want})
            pos[rid] += n
            if pos[rid] == len(seqs[rid]):
                ended.append(rid)
                running.remove(rid)
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def wanted_positions(steps, rid) -> List[int]:
    """The positions of request ``rid`` whose logits the trace asks for, in order."""
    out, p = [], 0
    for s in steps:
        for e in s["entries"]:
            if e["id"] == rid:
                out.extend(p + w for w in e["want"])
                p += len(e["tokens"])
    return out


def max_live_tokens(steps, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each request rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def replay(engine, steps) -> Dict[str, torch.Tensor]:
    """Runs the steps through ``engine.step``; returns request -> logits [positions, vocab] (CPU)."""
    from pytriton_llama_b200.engine.engine import StepEntry
    rows: Dict[str, Dict[int, torch.Tensor]] = {}
    fed: Dict[str, int] = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        out = engine.step(entries)
        logits = out.logits.float().cpu() if out.logits is not None else None
        r = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                rows.setdefault(e["id"], {})[base + w] = logits[r]
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            engine.finish(rid)
            fed.pop(rid, None)
        engine.cache.check_invariants()
    return {rid: torch.stack([d[p] for p in sorted(d)]) for rid, d in rows.items()}
