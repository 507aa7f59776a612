"""A decoder-only model assembled from a ``ModelSpec``: embedding, blocks run in the listed order,
final norm and LM head on the wanted rows only.

lite_llama/models/llama.py:189-223 is the same pipeline for one architecture with the LM head
over every position (:221); here only the rows whose logits are asked for reach the head.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import CacheNeed, Part, Runtime, TensorSpec, build_part
from .spec import ModelSpec


def _walk(part: Part, spec, prefix: str = ""):
    """Yields (part, spec) of a part and all parts nested in it."""
    yield part, spec
    for name, child in part.children().items():
        yield from _walk(child, spec.parts[name])


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = runtime
        self.blocks = [build_part("block", b, runtime) for b in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ tensors
    def expected_tensors(self) -> Dict[str, TensorSpec]:
        """Checkpoint name -> spec of every tensor the model reads."""
        out: Dict[str, TensorSpec] = {
            self.spec.embedding: TensorSpec((self.spec.vocab_size, self.spec.hidden_size)),
        }
        if self.spec.lm_head is not None:
            out[self.spec.lm_head] = TensorSpec((self.spec.vocab_size, self.spec.hidden_size))
        roots = [(b, s) for b, s in zip(self.blocks, self.spec.layers)] + [(self.final_norm, self.spec.final_norm)]
        for root, rspec in roots:
            for part, pspec in _walk(root, rspec):
                for local, ts in part.tensor_specs().items():
                    out[pspec.tensors[local]] = ts
        return out

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """``tensors``: checkpoint name -> CPU tensor, already checked against ``expected_tensors``."""
        rt = self.rt
        self.embedding = tensors[self.spec.embedding].to(device=rt.device, dtype=rt.dtype).contiguous()
        if self.spec.lm_head is None:
            self.lm_head = self.embedding
        else:
            self.lm_head = tensors[self.spec.lm_head].to(device=rt.device, dtype=rt.dtype).contiguous()
        roots = [(b, s) for b, s in zip(self.blocks, self.spec.layers)] + [(self.final_norm, self.spec.final_norm)]
        for root, rspec in roots:
            for part, pspec in _walk(root, rspec):
                specs = part.tensor_specs()
                if specs:
                    part.load({local: tensors.get(pspec.tensors[local]) for local in specs})

    # ------------------------------------------------------------------ cache
    def cache_entries(self) -> Dict[int, CacheNeed]:
        """Cache entry id -> what the layer that writes it needs."""
        out: Dict[int, CacheNeed] = {}
        for e in self.spec.run_order:
            need = self.blocks[e.layer].cache_need()
            if e.cache in out and out[e.cache].group_key() != need.group_key():
                raise ValueError(f"cache entry {e.cache} is used by layers with different needs")
            out.setdefault(e.cache, need)
        return out

    # ------------------------------------------------------------------ forward
    def forward(self, token_ids: torch.Tensor, ctx, cache_views, logit_rows: Optional[torch.Tensor]):
        """token_ids int32 [T]; ``cache_views(entry, write)`` gives the LayerCacheView of a run;
        returns float32 logits [len(logit_rows), vocab] (None when no row is wanted)."""
        ops = self.rt.ops
        begin = getattr(ops, "begin_forward", None)
        if begin is not None:
            begin()             # (what an operator set keeps per step, such as rotary angles, starts afresh)
        x = ops.embed(token_ids, self.embedding)
        residual = None
        run = self.spec.run_order
        for i, e in enumerate(run):
            block = self.blocks[e.layer]
            kw = {}
            if i + 1 < len(run) and getattr(block, "takes_next_norm", False):
                # the norm that reads the residual after this block (the final norm selects rows and does its own work)
                kw["next_norm"] = getattr(self.blocks[run[i + 1].layer], "norm1", None)
            x, residual = block.forward(x, residual, ctx, cache_views(e.cache, e.write), **kw)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        y, _ = self.final_norm.forward(x, residual, rows=logit_rows)
        return ops.linear(y, self.lm_head, out_dtype=torch.float32)
