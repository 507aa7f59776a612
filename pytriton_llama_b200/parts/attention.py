"""Grouped-query attention over the paged cache.

lite_llama/models/llama.py:26-105: q/k/v projections without bias (k and v fused in one weight,
:23,76), head-major split, rotary encoding of q and k, keys and values stored in the cache after
the rotation (:46-51), softmax(q k^T / sqrt(d)) v with query head h reading kv head h // group
(lite_llama/kernels/flashattentionv2.py:108), output projection.  lite_llama has one path for
prompts and one for single tokens; here one call serves any mix: the step's keys and values are
written to their pages first, then every token attends over the pages up to its own position.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from .base import CacheNeed, Part, PartSpec, Runtime, TensorSpec, build_part, register_part


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    """params: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, optional ``window`` (keys kept per
    query, 0 = all) and ``scale``.  Nested part ``position``.
    Tensors: ``q`` [heads*d, hidden], ``k``, ``v`` [kv_heads*d, hidden], ``o`` [hidden, heads*d]."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.window = int(p.get("window") or 0)
        self.scale = float(p.get("scale") or 1.0 / math.sqrt(self.head_dim))
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are no multiple of {self.kv_heads} kv heads")
        if self.head_dim % 16:
            raise ValueError(f"head size {self.head_dim}: the attention kernels take multiples of 16")
        self.position = build_part("position", spec.parts["position"], runtime)
        self.w_qkv = None
        self.w_o = None

    def children(self):
        return {"position": self.position}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        d = self.head_dim
        return {
            "q": TensorSpec((self.heads * d, self.hidden)),
            "k": TensorSpec((self.kv_heads * d, self.hidden)),
            "v": TensorSpec((self.kv_heads * d, self.hidden)),
            "o": TensorSpec((self.hidden, self.heads * d)),
        }

    def load(self, tensors) -> None:
        # one [ (heads + 2 kv_heads) d, hidden ] weight: q rows, then k, then v (the k|v part is
        # lite_llama's kv_proj_weight, lite_llama/executor/weight_convert.py:229-246)
        self.w_qkv = self._to_compute(torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0))
        self.w_o = self._to_compute(tensors["o"])

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="window" if self.window else "full", kv_heads=self.kv_heads,
                         head_dim=self.head_dim, window=self.window)

    fuses_residual = True   # forward() may add its output into the residual itself and return None
    accepts_normed = True   # x may be a norm's prepared input (the q|k|v product finishes the norm)
    emits_normed = True     # the output product may prepare the input of the norm that follows

    def forward(self, x, ctx, cache, residual=None, next_norm=None):
        ops = self.rt.ops
        table = self.position.rotary_table()
        g = cache.group
        whole = getattr(ops, "projected_rope_attention", None)      # an operator set may run projection, rotation and attention as one
        both = getattr(ops, "rope_attention", None)                 # ... or rotation and attention
        qkv = None
        if table is None:
            # The encoding is no rotation of (j, j + rot/2) pairs by a table of frequencies: it turns
            # q and k itself (in place, in the projection's output), and the kernels that follow only
            # store k and v and attend.
            qkv = ops.linear(x, self.w_qkv)
            qk_width = (self.heads + self.kv_heads) * self.head_dim
            self.position.apply(qkv[:, :qk_width], ctx.positions, self.heads + self.kv_heads, self.head_dim)
            inv_freq, rot, whole = None, 0, None
        else:
            inv_freq, rot = table
        if whole is not None:
            o = whole(x, self.w_qkv, ctx.positions, inv_freq, rot, g.slots, cache.kv, g.block_table, ctx.tok_req, self.heads,
                      self.kv_heads, self.head_dim, g.page_size, self.scale, window=self.window,
                      splits=ctx.attn_splits, hints=ctx, write=cache.write)
        elif both is not None:
            if qkv is None:
                qkv = ops.linear(x, self.w_qkv)
            o = both(qkv, ctx.positions, inv_freq, rot, g.slots, cache.kv, g.block_table, ctx.tok_req, self.heads,
                     self.kv_heads, self.head_dim, g.page_size, self.scale, window=self.window,
                     splits=ctx.attn_splits, hints=ctx, write=cache.write)
        else:
            if qkv is None:
                qkv = ops.linear(x, self.w_qkv)
            ops.rope_kv_write(qkv, ctx.positions, inv_freq, rot, g.slots if cache.write else None,
                              cache.kv if cache.write else None, self.heads, self.kv_heads, self.head_dim,
                              g.page_size)
            o = ops.paged_attention(qkv, cache.kv, g.block_table, ctx.tok_req, ctx.positions, self.heads,
                                    self.kv_heads, self.head_dim, g.page_size, self.scale, window=self.window,
                                    splits=ctx.attn_splits, hints=ctx)
        if residual is not None:
            if next_norm is not None and getattr(ops, "fuses_next_norm", False):
                return ops.linear_add(o, self.w_o, residual, next_norm=next_norm)
            return ops.linear_add(o, self.w_o, residual)      # None when the product's epilogue did the add
        return ops.linear(o, self.w_o)
