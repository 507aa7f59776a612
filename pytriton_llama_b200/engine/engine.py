"""The engine: a loaded model, its cache, and ONE step function.

lite_llama's executor (lite_llama/executor/model_executor.py:38-72,183-208,314-320) builds the
model, loads weights, sizes the cache and exposes ``forward(input_ids, prev_pos)`` for a padded
batch that is either all prompt or all single tokens.  ``Engine.step`` takes a batch of
(request, its next tokens): portions of prompts beside single decoded tokens, cut anywhere.  It
runs only those tokens, as one batch, against the cache that earlier steps left, and returns the
float32 logits at the wanted places.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Hashable, List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages
from ..config.engine import EngineConfig
from ..config.registry import read_config_json, resolve_architecture
from ..models.decoder import DecoderModel
from ..parts.base import Runtime
from ..weights.loader import check_tensors
from ..weights.safetensors_io import read_folder
from ..ops.worklists import PAD_TOKEN_ROW, StepWork
from .context import GroupStepView, LayerCacheView, StepContext


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    from_row: Optional[int] = None    # the single token is ``Engine.sampled[from_row]``, read on the device


@dataclass
class StepOutput:
    logits: Optional[torch.Tensor]            # float32 [wanted, vocab], in the order of entries and of want
    rows: List[tuple] = field(default_factory=list)   # (request, index within its tokens) of each logits row
    num_tokens: int = 0
    num_requests: int = 0
    pages_used: int = 0                       # pages held after this step, over all groups of cache entries
    pages_free: int = 0
    step_ms: Optional[float] = None           # device time of the step (CUDA events); with ``EngineConfig.timing`` only
    kernel_ms: Optional[Dict[str, float]] = None      # ... and by class of kernels, where the operator set reports it


@dataclass
class EngineStats:
    """Running totals over the steps of an engine (``Engine.stats``)."""
    steps: int = 0
    tokens: int = 0
    wanted_rows: int = 0
    peak_pages_used: int = 0
    step_ms: float = 0.0                      # timed steps only
    timed_steps: int = 0
    kernel_ms: Dict[str, float] = field(default_factory=dict)

    def add(self, out: "StepOutput") -> None:
        self.steps += 1
        self.tokens += out.num_tokens
        self.wanted_rows += len(out.rows)
        self.peak_pages_used = max(self.peak_pages_used, out.pages_used)
        if out.step_ms is not None:
            self.step_ms += out.step_ms
            self.timed_steps += 1
        for k, v in (out.kernel_ms or {}).items():
            self.kernel_ms[k] = self.kernel_ms.get(k, 0.0) + v

    def summary(self) -> Dict[str, object]:
        d = {"steps": self.steps, "tokens": self.tokens, "wanted_rows": self.wanted_rows, "peak_pages_used": self.peak_pages_used}
        if self.timed_steps:
            d["step_ms_mean"] = round(self.step_ms / self.timed_steps, 4)
            d["tokens_per_s_device"] = round(self.tokens / (self.step_ms * 1e-3), 1) if self.step_ms > 0 else None
            d["kernel_ms"] = {k: round(v, 3) for k, v in sorted(self.kernel_ms.items())}
        return d


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class _HostBatch:
    """A step's requests as host lists, before they are packed for the device."""

    def __init__(self, entries, q_lens, starts, fresh, state_slots, slots_by_group, logit_rows, work=None):
        self.entries, self.q_lens, self.starts, self.fresh = entries, q_lens, starts, fresh
        self.state_slots, self.slots_by_group, self.logit_rows = state_slots, slots_by_group, logit_rows
        self.takes_sampled = any(e.from_row is not None for e in entries)
        self.R = len(entries)
        self.T = sum(q_lens)
        self.max_q_len = max(q_lens)
        self.max_ctx_len = max(s + n for s, n in zip(starts, q_lens))
        self.work: Dict[str, List[int]] = work or {}      # the operator set's lists for this step (ops.plan_step)


class _Layout:
    """Where each integer array of a step lies inside one packed int32 buffer (one copy per step)."""

    def __init__(self, T: int, R: int, M: int, bt_width: int, groups: List[int], static_rows: bool = False,
                 work_sizes: Optional[Dict[str, int]] = None):
        self.T, self.R, self.M, self.bt_width, self.groups, self.static_rows = T, R, M, bt_width, groups, static_rows
        self.work_sizes = dict(work_sizes or {})           # integers each of the operator set's lists may hold
        self.seg: Dict[str, tuple] = {}
        cursor = 0
        names = [("tokens", T), ("token_src", T), ("positions", T), ("tok_req", T), ("q_start", R + 1), ("ctx_len", R),
                 ("state_slot", R), ("fresh", R), ("logit_rows", M)]
        names += [(f"work:{name}", n) for name, n in sorted(self.work_sizes.items())]
        for g in groups:
            names += [(f"slots{g}", T), (f"bt{g}", R * bt_width)]
        for name, n in names:
            self.seg[name] = (cursor, n)
            cursor += _pad4(max(n, 1))
        self.size = cursor

    def view(self, dev: torch.Tensor, name: str) -> torch.Tensor:
        lo, n = self.seg[name]
        return dev[lo:lo + n]


@dataclass(frozen=True)
class _DecodeShape:
    """Names the captured step of ``batch`` single tokens whose contexts are at most ``context`` tokens
    long, where that is less than the engine's longest (the captured step for the longest has the
    plain batch size as its name)."""
    batch: int
    context: int


@dataclass
class _DecodeGraph:
    graph: object
    layout: _Layout
    staging: list          # ring of (pinned host buffer, event recorded after its last copy)
    dev: torch.Tensor
    logits: torch.Tensor
    launches: int
    turn: int = 0
    last_used: int = 0


class Engine:
    def __init__(self, model_dir: Union[str, Path, None], config: Optional[EngineConfig] = None,
                 device: Union[str, torch.device] = "cuda:0", ops=None, model_config: Optional[dict] = None,
                 random_seed: Optional[int] = None):
        """Loads the model of ``model_dir`` (config.json + safetensors).  With ``model_dir`` None,
        ``model_config`` (the content of a config.json) and ``random_seed`` build the same model
        with random weights drawn on the device, without writing a folder."""
        self.config = config or EngineConfig()
        self.device = torch.device(device)
        raw = read_config_json(model_dir) if model_dir is not None else dict(model_config)
        arch = resolve_architecture(raw)
        self.model_config = arch.config_from_dict(raw)
        spec = arch.spec_from_config(self.model_config)
        if ops is None:
            from ..ops.cuda import CudaOps
            ops = CudaOps(self.device)
        self.ops = ops
        self.runtime = Runtime(self.device, self.config.dtype, ops)
        self.model = DecoderModel(spec, self.runtime)
        if model_dir is not None:
            tensors = read_folder(model_dir)
            ignorable = ["lm_head.weight"] if spec.lm_head is None else []
            check_tensors(self.model.expected_tensors(), tensors, ignorable=ignorable)
        else:
            from ..weights.random_init import random_tensors_on_device
            tensors = random_tensors_on_device(self.model.expected_tensors(), int(random_seed or 0),
                                               spec.initializer_range, self.config.dtype, self.device)
        self.model.load(tensors)
        del tensors
        self.vocab_size = spec.vocab_size
        self.eos_token_ids = list(spec.eos_token_ids)
        self.memory_report: Optional[dict] = None      # filled when the pool is sized from free memory
        entries = self.model.cache_entries()
        num_pages = self.config.max_gpu_num_blocks or self._pages_from_free_memory(entries)
        self.cache = CacheManager(entries, self.config.page_size, num_pages, self.config.max_num_seqs,
                                  self.config.max_seq_len, self.device, self.config.dtype)
        self._pinned = self.device.type == "cuda"
        # Tokens sampled from the last step's logits rows, for callers that sample on the device and
        # launch the next step before they have read them: an entry with ``from_row`` takes its
        # token from here.
        self.sampled = torch.zeros(max(1, self.config.max_num_seqs), dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self.stats = EngineStats()
        if self.config.timing and hasattr(self.ops, "enable_timing"):
            self.ops.enable_timing()
        self._graphs = {}          # captured steps: padded batch size or _DecodeShape (single tokens only), or a shape tuple
        self._shape_seen: Dict[tuple, int] = {}
        self._shape_captures = 0
        self._graph_pool = None    # one memory pool for the captured steps of mixed shapes

    # ------------------------------------------------------------------ sizing
    def _pages_from_free_memory(self, entries) -> int:
        """Pages that fit into ``gpu_memory_fraction`` of the memory still free after the weights
        (lite_llama/executor/mem_manager.py:98-108 sizes its pool the same way), capped at what
        ``max_num_seqs`` requests of ``max_seq_len`` tokens can ever hold."""
        esize = torch.empty((), dtype=self.config.dtype).element_size()
        per_page: Dict[tuple, int] = {}
        for need in entries.values():
            if need.kind in ("full", "window"):
                k = need.group_key()
                per_page[k] = per_page.get(k, 0) + 2 * need.kv_heads * need.head_dim * self.config.page_size * esize
        if not per_page:
            return 1
        bytes_per_page = sum(per_page.values())   # one page in every group
        cap = self.config.max_num_seqs * -(-self.config.max_seq_len // self.config.page_size)
        if self.device.type != "cuda":
            return cap
        free, total = torch.cuda.mem_get_info(self.device)
        workspace = 2 << 30
        fit = int((free * self.config.gpu_memory_fraction - workspace) // bytes_per_page)
        pages = min(cap, fit)
        # what lite_llama prints when it sizes its pool (lite_llama/executor/mem_manager.py:112-123), kept for callers
        self.memory_report = {"device_total_gb": round(total / 2 ** 30, 2), "free_after_weights_gb": round(free / 2 ** 30, 2),
                              "fraction": self.config.gpu_memory_fraction, "bytes_per_page_all_groups": bytes_per_page,
                              "pages_that_fit": fit, "pages_ever_needed": cap, "pages": pages,
                              "cache_gb": round(max(pages, 0) * bytes_per_page / 2 ** 30, 3)}
        logging.getLogger(__name__).info("cache pool sized from free memory: %s", self.memory_report)
        if fit <= 0:
            raise OutOfPages("no memory left for the cache after loading the weights")
        return pages

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], validate: bool = True, own_logits: bool = True) -> StepOutput:
        """``validate=False`` skips the checks of tokens, wanted places and free pages for callers
        that made them already (the scheduler's plans).  The logits of a step that ran from a captured
        graph lie in memory that the next captured step writes again; they are copied out of it unless
        ``own_logits=False`` says that the caller is done with them before its next step (the
        generation loop, which samples at once)."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return StepOutput(None, [], 0)
        cache = self.cache
        seen = set()
        for e in entries if validate else ():
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            toks = np.asarray(e.tokens)
            if e.from_row is not None:
                if len(e.tokens) != 1 or not 0 <= int(e.from_row) < self.sampled.shape[0]:
                    raise ValueError(f"request {e.request!r}: from_row names one sampled token, row 0..{self.sampled.shape[0] - 1}")
            elif toks.size and (int(toks.min()) < 0 or int(toks.max()) >= self.vocab_size):
                raise ValueError(f"a token of request {e.request!r} is outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.request!r} wants logits at {w} but brings {len(e.tokens)} tokens")
            have = cache.tokens_of(e.request) if cache.has(e.request) else 0
            if have + len(e.tokens) > self.config.max_seq_len:
                raise ValueError(f"request {e.request!r} would reach {have + len(e.tokens)} tokens; max_seq_len is {self.config.max_seq_len}")
        if validate and not cache.can_append([(e.request, len(e.tokens)) for e in entries]):
            raise OutOfPages("the cache cannot hold this step's tokens")

        q_lens = [len(e.tokens) for e in entries]
        fresh, starts, slots_by_group, state_slots = [], [], {}, []
        for e in entries:
            if not cache.has(e.request):
                cache.admit(e.request)
                fresh.append(1)
            else:
                fresh.append(1 if cache.tokens_of(e.request) == 0 else 0)
            starts.append(cache.tokens_of(e.request))
            for g, sl in cache.append(e.request, len(e.tokens)).items():
                slots_by_group.setdefault(g, []).extend(sl)
            state_slots.append(cache.slot_of(e.request))
        rows, logit_rows = [], []
        base = 0
        for e, n in zip(entries, q_lens):
            for w in e.want:
                rows.append((e.request, int(w)))
                logit_rows.append(base + int(w))
            base += n
        plan = getattr(self.ops, "plan_step", None)
        batch = _HostBatch(entries, q_lens, starts, fresh, state_slots, slots_by_group, logit_rows,
                           work=plan(q_lens, starts) if plan is not None else None)
        self.steps_run += 1
        timing = self.config.timing and self.device.type == "cuda"
        if timing:
            t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t_start.record()
        bucket = self._graph_bucket(batch)
        if bucket:
            logits = self._run_graph(bucket, batch)
            if isinstance(bucket, tuple):
                logits = logits[:len(logit_rows)] if logit_rows else None      # the wanted rows, in order
            elif logit_rows != list(range(len(entries))):
                idx = torch.tensor(logit_rows, dtype=torch.long, device=self.device)
                logits = logits.index_select(0, idx) if logit_rows else None
            if logits is not None and own_logits and logits._base is not None:
                logits = logits.clone()       # out of the captured step's memory, which the next replay writes again
        else:
            layout = _Layout(batch.T, batch.R, len(logit_rows), self._table_width(batch), self._paged_groups(),
                             work_sizes={name: len(v) for name, v in batch.work.items()})
            host = torch.empty(layout.size, dtype=torch.int32, pin_memory=self._pinned)
            self._fill(host.numpy(), layout, batch)
            dev = host.to(self.device, non_blocking=True)
            if batch.takes_sampled:
                self.ops.take_tokens(layout.view(dev, "tokens"), layout.view(dev, "token_src"), self.sampled)
            ctx, cache_view = self._context(dev, layout, batch.q_lens, [s + n for s, n in zip(starts, q_lens)],
                                            self._choose_splits(batch.T, max(s + n for s, n in zip(starts, q_lens))),
                                            work_items=self._work_items(batch.work),
                                            in_order=self._work_in_order(batch.work, batch.T))
            logits = self.model.forward(layout.view(dev, "tokens"), ctx, cache_view,
                                        layout.view(dev, "logit_rows") if logit_rows else None)
        out = StepOutput(logits, rows, batch.T, batch.R)
        for g in self._paged_groups():
            free = cache.free_pages(g)
            out.pages_free += free
            out.pages_used += cache.groups[g].pool.num_pages - free
        if timing:
            t_end.record()
            t_end.synchronize()
            out.step_ms = t_start.elapsed_time(t_end)
            take = getattr(self.ops, "take_timings", None)
            out.kernel_ms = take() if take is not None else None
        self.stats.add(out)
        return out

    # ------------------------------------------------------------------ batch assembly
    def _paged_groups(self) -> List[int]:
        return [g for g, grp in enumerate(self.cache.groups) if grp.paged]

    def _table_width(self, batch: "_HostBatch") -> int:
        widths = [len(self.cache.block_table_array(e.request, g)) for g in self._paged_groups() for e in batch.entries]
        return _pad4(max([1] + widths))

    def _fill(self, h: np.ndarray, layout: "_Layout", b: "_HostBatch") -> None:
        """Writes the step's integers into the packed host buffer; rows beyond the batch (a padded
        graph bucket) get request -1 and slot -1, which every kernel skips."""
        T, R = b.T, b.R

        def put(name, values, fill=0):
            lo, n = layout.seg[name]
            h[lo:lo + len(values)] = values
            h[lo + len(values):lo + n] = fill

        put("tokens", np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in b.entries]))
        lo, n = layout.seg["token_src"]
        h[lo:lo + n] = -1
        if b.takes_sampled:
            t0 = 0
            for e, k in zip(b.entries, b.q_lens):
                if e.from_row is not None:
                    h[lo + t0] = e.from_row
                    h[layout.seg["tokens"][0] + t0] = 0
                t0 += k
        put("positions", np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(b.starts, b.q_lens)]))
        put("tok_req", np.repeat(np.arange(R, dtype=np.int32), b.q_lens), fill=-1)
        put("q_start", np.concatenate([[0], np.cumsum(b.q_lens)]).astype(np.int32), fill=T)
        put("ctx_len", [s + n for s, n in zip(b.starts, b.q_lens)])
        put("state_slot", b.state_slots)
        put("fresh", b.fresh)
        lo, n = layout.seg["logit_rows"]
        if layout.static_rows:
            h[lo:lo + n] = np.arange(n, dtype=np.int32)
        elif n:
            put("logit_rows", b.logit_rows)          # (a padded shape asks for row 0 again in the rows it has too many)
        # The operator set's lists.  A captured step has room for more items than the step brings:
        # the rest is padding, either a number or a token row that belongs to no request (the
        # shape is chosen so that there is one).
        infos = self._work_lists()
        for name in layout.work_sizes:
            values = b.work.get(name, ())
            if len(values) > layout.work_sizes[name]:
                raise RuntimeError(f"work list {name!r} has {len(values)} integers, the captured step holds {layout.work_sizes[name]}")
            pad = infos[name].pad if name in infos else 0
            put(f"work:{name}", values, fill=min(T, layout.T - 1) if pad == PAD_TOKEN_ROW else pad)
        for g in layout.groups:
            put(f"slots{g}", b.slots_by_group[g], fill=-1)
            lo, n = layout.seg[f"bt{g}"]
            bt = h[lo:lo + n].reshape(layout.R, layout.bt_width)
            bt.fill(-1)
            for i, e in enumerate(b.entries):
                t = self.cache.block_table_array(e.request, g)
                bt[i, :len(t)] = t

    def _work_lists(self) -> dict:
        """name -> ``WorkList`` of the lists the operator set wants packed with a step."""
        return getattr(self.ops, "WORK_LISTS", {})

    def _work_items(self, work: Dict[str, List[int]]) -> Dict[str, int]:
        infos = self._work_lists()
        return {name: len(v) // (infos[name].width if name in infos else 1) for name, v in work.items()}

    def _work_in_order(self, work: Dict[str, List[int]], T: int) -> Dict[str, bool]:
        infos = self._work_lists()
        return {name: (name not in infos or infos[name].width == 1) and len(v) == T and list(v) == list(range(T))
                for name, v in work.items()}

    def _context(self, dev: torch.Tensor, layout: "_Layout", q_lens, ctx_lens, splits: int, work_items: Dict[str, int],
                 in_order: Dict[str, bool]):
        cache = self.cache
        infos = self._work_lists()
        work = {name: StepWork(layout.view(dev, f"work:{name}")[:n * (infos[name].width if name in infos else 1)], n,
                               bool(in_order.get(name, False)))
                for name, n in work_items.items()}
        groups = {g: GroupStepView(page_size=cache.page_size,
                                   block_table=layout.view(dev, f"bt{g}").view(layout.R, layout.bt_width),
                                   slots=layout.view(dev, f"slots{g}"), window=cache.groups[g].need.window)
                  for g in layout.groups}
        ctx = StepContext(num_tokens=layout.T, num_requests=layout.R, positions=layout.view(dev, "positions"),
                          tok_req=layout.view(dev, "tok_req"), q_start=layout.view(dev, "q_start"),
                          ctx_len=layout.view(dev, "ctx_len"), state_slot=layout.view(dev, "state_slot"),
                          fresh=layout.view(dev, "fresh"), groups=groups, q_lens=list(q_lens),
                          ctx_lens=list(ctx_lens), max_q_len=max(q_lens), max_ctx_len=max(ctx_lens),
                          attn_splits=splits, work=work)

        def cache_view(entry: int, write: bool) -> LayerCacheView:
            g = cache.entry_group[entry]
            grp = cache.groups[g]
            return LayerCacheView(group=groups.get(g), kv=grp.kv.get(entry), state=grp.state.get(entry), write=write)
        return ctx, cache_view

    def _choose_splits(self, tokens: int, max_ctx: int) -> int:
        """Key-range splits for steps with few tokens and long contexts (more parallel work)."""
        if tokens > 64 or max_ctx < 512:
            return 1
        return int(min(32, max(1, max_ctx // 256)))

    # ------------------------------------------------------------------ steps from CUDA graphs
    def _graph_bucket(self, batch: "_HostBatch"):
        """What names the captured graph that can run this step, or 0: the padded batch size for a
        step of single tokens (lite_llama captures its decode step for batch sizes 1, 2, 4, 8, 16,
        ...: lite_llama/executor/cuda_graph.py:6-7,113-132), a padded shape (a tuple) for a step that
        holds prompt portions.  Only for models whose mixers keep nothing but paged keys and values."""
        if not self.config.compiled_model or self.device.type != "cuda" or self.config.timing:
            return 0          # (timing brackets every operator with events, which a capture cannot hold)
        if any(not grp.paged or grp.state for grp in self.cache.groups):
            return 0
        if batch.max_q_len != 1:
            return self._shape_bucket(batch) if self.config.capture_mixed_steps else 0
        b = 1
        while b < batch.R:
            b *= 2
        if b > max(64, self.config.max_num_seqs):
            return 0
        context = self._context_bucket(batch.max_ctx_len)
        return b if context >= self.config.max_seq_len else _DecodeShape(b, context)

    def _context_bucket(self, longest: int) -> int:
        """The context length a captured step of single tokens is made for: the operator set decides
        once, at capture, how it cuts the keys of a request into parallel work, and what suits
        131,072 keys is slow for 2,000.  So steps are captured per class of context length
        (``graph_context_buckets``; classes that reach within a factor of two of ``max_seq_len`` fall
        into the last, which is ``max_seq_len`` itself)."""
        for c in self.config.graph_context_buckets:
            if longest <= c and 2 * c <= self.config.max_seq_len:
                return c
        return self.config.max_seq_len

    GRAPH_MAX_TOKENS = 1024      # larger steps keep the GPU busy for longer than the host needs to launch them
    GRAPH_MAX_SHAPES = 24
    GRAPH_MAX_CAPTURES = 96      # a workload that keeps cycling through more shapes than are kept stops capturing new ones

    def _shape_bucket(self, batch: "_HostBatch"):
        """Steps with prompt portions of up to 1,024 tokens are bound by the host's launches (about
        11 us each, twice the GPU's time at 300 tokens), so they run from captured graphs too: the
        step's shape is padded to (tokens, requests, wants logits, items of each of the operator
        set's work lists) with few values each, and a shape that comes a second time is captured.
        Padded token rows have request -1 and slot -1, padded list items are what the operator set
        says they must be: every kernel skips them."""
        T, R, M = batch.T, batch.R, len(batch.logit_rows)
        if T > self.GRAPH_MAX_TOKENS:
            return 0
        pow2 = lambda n: 0 if n == 0 else 1 << (n - 1).bit_length()
        step = 64 if T <= 256 else 128
        t_pad = -(-T // step) * step
        lists, needs_free_row = [], False
        for name, info in sorted(self._work_lists().items()):
            items = len(batch.work.get(name, ())) // info.width
            padded = pow2(-(-items // info.group)) * info.group     # whole groups, a power of two of them
            lists.append((name, padded))
            needs_free_row |= padded > items and info.pad == PAD_TOKEN_ROW
        if needs_free_row and t_pad == T:
            t_pad += step                                   # the padded items need a token row that belongs to no request
        r_pad = pow2(R)
        if M > r_pad:
            return 0                                        # (a replay that wants many rows of a prompt)
        shape = (t_pad, r_pad, 1 if M else 0, tuple(lists))
        if shape in self._graphs:
            return shape
        if self._shape_captures >= self.GRAPH_MAX_CAPTURES:
            return 0                                        # capturing costs tens of milliseconds: not again and again
        seen = self._shape_seen.get(shape, 0) + 1
        self._shape_seen[shape] = seen
        if len(self._shape_seen) > 4096:
            self._shape_seen.clear()
        return shape if seen >= 2 else 0

    def _run_graph(self, bucket, batch: "_HostBatch") -> torch.Tensor:
        g = self._graphs.get(bucket)
        if g is None:
            if isinstance(bucket, tuple):
                shapes = [k for k in self._graphs if isinstance(k, tuple)]
                if len(shapes) >= self.GRAPH_MAX_SHAPES:    # drop the shape that was used longest ago
                    del self._graphs[min(shapes, key=lambda k: self._graphs[k].last_used)]
                self._shape_captures += 1
            g = self._graphs[bucket] = self._capture(bucket)
        g.last_used = self.steps_run
        # The copy below is asynchronous: a staging buffer may be rewritten only after the copy that
        # last read it has finished, so each buffer of the ring carries an event.
        host, event = g.staging[g.turn % len(g.staging)]
        g.turn += 1
        event.synchronize()
        self._fill(host.numpy(), g.layout, batch)
        g.dev.copy_(host, non_blocking=True)
        event.record(torch.cuda.current_stream(self.device))
        g.graph.replay()
        if hasattr(self.ops, "launches"):
            self.ops.launches += g.launches
        if g.logits is None or isinstance(bucket, tuple):
            return g.logits
        return g.logits[:batch.R]

    def _capture(self, bucket) -> "_DecodeGraph":
        """Captures the step of a padded batch of single tokens (``bucket`` an int) or of a padded
        shape (a tuple, see ``_shape_bucket``).  While it is captured every token row belongs to no
        request, so the runs that record it touch no page of the cache."""
        width = _pad4(self.cache.max_blocks)
        infos = self._work_lists()
        longest = self.config.max_seq_len                    # what the step's kernels are laid out for
        if isinstance(bucket, tuple):
            t_pad, r_pad, wants, lists = bucket
            work_items = dict(lists)
            in_order = {}
            layout = _Layout(t_pad, r_pad, r_pad if wants else 0, width, self._paged_groups(),
                             work_sizes={name: n * infos[name].width for name, n in lists})
            q_lens = [t_pad] + [1] * (r_pad - 1)
        else:
            if isinstance(bucket, _DecodeShape):
                bucket, longest = bucket.batch, bucket.context
            plan = getattr(self.ops, "plan_step", None)
            work = plan([1] * bucket, [0] * bucket) if plan is not None else {}
            work_items, in_order = self._work_items(work), self._work_in_order(work, bucket)
            layout = _Layout(bucket, bucket, bucket, width, self._paged_groups(), static_rows=True,
                             work_sizes={name: len(v) for name, v in work.items()})
            q_lens, wants = [1] * bucket, 1
        host = torch.empty(layout.size, dtype=torch.int32, pin_memory=True)
        h = host.numpy()
        h.fill(0)
        for name, fill in [("tok_req", -1), ("token_src", -1)] + [(f"slots{g}", -1) for g in layout.groups] + [(f"bt{g}", -1) for g in layout.groups]:
            lo, n = layout.seg[name]
            h[lo:lo + n] = fill
        if layout.static_rows:
            lo, n = layout.seg["logit_rows"]
            h[lo:lo + n] = np.arange(n, dtype=np.int32)
            for name, values in work.items():
                lo, n = layout.seg[f"work:{name}"]
                h[lo:lo + n] = np.asarray(values, dtype=np.int32)
        dev = host.to(self.device)
        splits = self._choose_splits(layout.T, longest)
        ctx, cache_view = self._context(dev, layout, q_lens, [longest] * layout.R, splits,
                                        work_items=work_items, in_order=in_order)

        def run():
            self.ops.take_tokens(layout.view(dev, "tokens"), layout.view(dev, "token_src"), self.sampled)
            return self.model.forward(layout.view(dev, "tokens"), ctx, cache_view,
                                      layout.view(dev, "logit_rows") if wants else None)
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):      # libraries set themselves up outside the capture
                run()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = getattr(self.ops, "launches", 0)
        pool = None
        if isinstance(bucket, tuple):                        # mixed shapes share one pool: only one of them runs at a time
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            pool = self._graph_pool
        with torch.cuda.graph(graph, pool=pool):
            logits = run()
        launches = getattr(self.ops, "launches", 0) - before
        staging = [(torch.empty(layout.size, dtype=torch.int32, pin_memory=True), torch.cuda.Event()) for _ in range(4)]
        return _DecodeGraph(graph, layout, staging, dev, logits, launches)

    def check_device_status(self) -> None:
        """Raises if a kernel reported a problem (synchronises the device; call it off the hot path)."""
        if hasattr(self.ops, "check_status"):
            self.ops.check_status()

    # ------------------------------------------------------------------ requests
    def finish(self, request: Hashable) -> None:
        """Gives back everything the request holds."""
        if self.cache.has(request):
            self.cache.release(request)

    def finish_all(self) -> None:
        self.cache.release_all()
