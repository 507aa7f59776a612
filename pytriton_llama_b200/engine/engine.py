"""The engine: a loaded model, its cache, and ONE step function.

lite_llama's executor (lite_llama/executor/model_executor.py:38-72,183-208,314-320) builds the
model, loads weights, sizes the cache and exposes ``forward(input_ids, prev_pos)`` for a padded
batch that is either all prompt or all single tokens.  ``Engine.step`` takes a batch of
(request, its next tokens): portions of prompts beside single decoded tokens, cut anywhere.  It
runs only those tokens, as one batch, against the cache that earlier steps left, and returns the
float32 logits at the wanted places.
"""
from __future__ import annotations

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
from .context import GroupStepView, LayerCacheView, StepContext


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepOutput:
    logits: Optional[torch.Tensor]            # float32 [wanted, vocab], in the order of entries and of want
    rows: List[tuple] = field(default_factory=list)   # (request, index within its tokens) of each logits row
    num_tokens: int = 0


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class Engine:
    def __init__(self, model_dir: Union[str, Path], config: Optional[EngineConfig] = None,
                 device: Union[str, torch.device] = "cuda:0", ops=None):
        self.config = config or EngineConfig()
        self.device = torch.device(device)
        raw = read_config_json(model_dir)
        arch = resolve_architecture(raw)
        self.model_config = arch.config_from_dict(raw)
        spec = arch.spec_from_config(self.model_config)
        if ops is None:
            from ..ops.cuda import CudaOps
            ops = CudaOps(self.device)
        self.ops = ops
        self.runtime = Runtime(self.device, self.config.dtype, ops)
        self.model = DecoderModel(spec, self.runtime)
        tensors = read_folder(model_dir)
        ignorable = ["lm_head.weight"] if spec.lm_head is None else []
        check_tensors(self.model.expected_tensors(), tensors, ignorable=ignorable)
        self.model.load(tensors)
        del tensors
        self.vocab_size = spec.vocab_size
        self.eos_token_ids = list(spec.eos_token_ids)
        entries = self.model.cache_entries()
        num_pages = self.config.max_gpu_num_blocks or self._pages_from_free_memory(entries)
        self.cache = CacheManager(entries, self.config.page_size, num_pages, self.config.max_num_seqs,
                                  self.config.max_seq_len, self.device, self.config.dtype)
        self._pinned = self.device.type == "cuda"
        self.steps_run = 0

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
        free, _ = torch.cuda.mem_get_info(self.device)
        workspace = 2 << 30
        fit = int((free * self.config.gpu_memory_fraction - workspace) // bytes_per_page)
        if fit <= 0:
            raise OutOfPages("no memory left for the cache after loading the weights")
        return min(cap, fit)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> StepOutput:
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return StepOutput(None, [], 0)
        cache = self.cache
        seen = set()
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise ValueError(f"token {t} of request {e.request!r} is outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.request!r} wants logits at {w} but brings {len(e.tokens)} tokens")
            have = cache.tokens_of(e.request) if cache.has(e.request) else 0
            if have + len(e.tokens) > self.config.max_seq_len:
                raise ValueError(f"request {e.request!r} would reach {have + len(e.tokens)} tokens; max_seq_len is {self.config.max_seq_len}")
        if not cache.can_append([(e.request, len(e.tokens)) for e in entries]):
            raise OutOfPages("the cache cannot hold this step's tokens")

        R = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
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
        ctx_lens = [s + n for s, n in zip(starts, q_lens)]
        paged_groups = [g for g, grp in enumerate(cache.groups) if grp.paged]
        tables = {g: [cache.block_table(e.request, g) for e in entries] for g in paged_groups}
        bt_width = _pad4(max([1] + [len(t) for g in paged_groups for t in tables[g]]))
        rows, logit_rows = [], []
        base = 0
        for e, n in zip(entries, q_lens):
            for w in e.want:
                rows.append((e.request, int(w)))
                logit_rows.append(base + int(w))
            base += n
        M = len(logit_rows)

        # one packed int32 buffer, one copy to the device
        seg = {}
        cursor = 0

        def reserve(name, n):
            nonlocal cursor
            seg[name] = (cursor, n)
            cursor += _pad4(max(n, 1))

        reserve("tokens", T); reserve("positions", T); reserve("tok_req", T)
        reserve("q_start", R + 1); reserve("ctx_len", R); reserve("state_slot", R); reserve("fresh", R)
        reserve("logit_rows", M)
        for g in paged_groups:
            reserve(f"slots{g}", T); reserve(f"bt{g}", R * bt_width)
        host = torch.empty(cursor, dtype=torch.int32, pin_memory=self._pinned)
        h = host.numpy()

        def put(name, values):
            lo, n = seg[name]
            h[lo:lo + n] = values

        put("tokens", np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries]))
        put("positions", np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(starts, q_lens)]))
        put("tok_req", np.repeat(np.arange(R, dtype=np.int32), q_lens))
        put("q_start", np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32))
        put("ctx_len", ctx_lens); put("state_slot", state_slots); put("fresh", fresh)
        if M:
            put("logit_rows", logit_rows)
        for g in paged_groups:
            put(f"slots{g}", slots_by_group[g])
            bt = np.full((R, bt_width), -1, dtype=np.int32)
            for i, t in enumerate(tables[g]):
                bt[i, :len(t)] = t
            put(f"bt{g}", bt.reshape(-1))
        dev = host.to(self.device, non_blocking=True)

        def view(name):
            lo, n = seg[name]
            return dev[lo:lo + n]

        groups = {g: GroupStepView(page_size=cache.page_size,
                                   block_table=view(f"bt{g}").view(R, bt_width), slots=view(f"slots{g}"),
                                   window=cache.groups[g].need.window) for g in paged_groups}
        max_ctx = max(ctx_lens)
        ctx = StepContext(num_tokens=T, num_requests=R, positions=view("positions"), tok_req=view("tok_req"),
                          q_start=view("q_start"), ctx_len=view("ctx_len"), state_slot=view("state_slot"),
                          fresh=view("fresh"), groups=groups, q_lens=q_lens, ctx_lens=ctx_lens,
                          max_q_len=max(q_lens), max_ctx_len=max_ctx,
                          attn_splits=self._choose_splits(T, max_ctx))

        def cache_view(entry: int, write: bool) -> LayerCacheView:
            g = cache.entry_group[entry]
            grp = cache.groups[g]
            return LayerCacheView(group=groups.get(g), kv=grp.kv.get(entry), state=grp.state.get(entry), write=write)

        logits = self.model.forward(view("tokens"), ctx, cache_view, view("logit_rows") if M else None)
        self.steps_run += 1
        return StepOutput(logits, rows, T)

    def _choose_splits(self, tokens: int, max_ctx: int) -> int:
        """Key-range splits for steps with few tokens and long contexts (more parallel work)."""
        if tokens > 64 or max_ctx < 512:
            return 1
        return int(min(32, max(1, max_ctx // 256)))

    # ------------------------------------------------------------------ requests
    def finish(self, request: Hashable) -> None:
        """Gives back everything the request holds."""
        if self.cache.has(request):
            self.cache.release(request)

    def finish_all(self) -> None:
        self.cache.release_all()
