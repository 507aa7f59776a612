"""What one step looks like to the parts: the flat batch on the device and the cache views.

A step carries ``T`` tokens of ``R`` requests, request after request.  Nothing in here says
whether a request is in its prompt or decoding: a portion is ``q_len`` new tokens that follow
``ctx_len - q_len`` tokens already in the cache.  (lite_llama hands its layers an ``AttentionInfo``
with the cache buffers, ``cur_select_index`` and ``b_req_tokens_table`` for the same purpose,
lite_llama/executor/executor_struct.py:13-23, and tells prompt from decode by the sequence length,
lite_llama/models/llama.py:62-118.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch


@dataclass
class GroupStepView:
    """Paging data of one cache group for this step."""
    page_size: int
    block_table: torch.Tensor   # int32 [R, max_pages]; -1 where a page was given back or never held
    slots: torch.Tensor         # int32 [T]; page * page_size + offset of each new token, -1 = do not store
    window: int = 0


@dataclass
class LayerCacheView:
    """The cache entry one run of a layer uses."""
    group: Optional[GroupStepView]
    kv: Optional[torch.Tensor]      # [pages, 2, kv_heads, page_size, head_dim] of this entry
    state: Optional[torch.Tensor]   # [slots, *state_shape] per-request state of this entry
    write: bool = True              # False: read what another run of a layer stored


@dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    positions: torch.Tensor        # int32 [T] position of each token in its request
    tok_req: torch.Tensor          # int32 [T] row of the token's request in this step
    q_start: torch.Tensor          # int32 [R + 1] first token of each request (prefix sums of q_len)
    ctx_len: torch.Tensor          # int32 [R] tokens of the request in the cache after this step
    state_slot: torch.Tensor       # int32 [R] slot of the request's fixed-size state
    fresh: torch.Tensor            # int32 [R] 1 if this portion starts the request (state must be reset)
    groups: Dict[int, GroupStepView] = field(default_factory=dict)
    q_lens: List[int] = field(default_factory=list)       # host copies for launch decisions
    ctx_lens: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_ctx_len: int = 0
    attn_splits: int = 1
    # integer lists the operator set asked for (``ops.plan_step``): name -> ``StepWork``
    work: Dict[str, Any] = field(default_factory=dict)
