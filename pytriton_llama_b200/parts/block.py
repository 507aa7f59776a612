"""How norm, mixer, norm and feed-forward sit around the residual stream.

lite_llama/models/llama.py:136-162: pre-norm block.  The stream is carried as two tensors: the
output of the last sub-layer (not yet added) and the float32 residual; each norm first adds the
former into the latter.  The block returns its feed-forward output un-added, so the next block's
first norm (or the model's final norm, :219) folds it in.
"""
from __future__ import annotations

from .base import Part, PartSpec, Runtime, build_part, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Part):
    """Nested parts: ``norm1``, ``mixer``, ``norm2``, ``ffn``."""

    def __init__(self, spec: PartSpec, runtime: Runtime):
        super().__init__(spec, runtime)
        self.norm1 = build_part("norm", spec.parts["norm1"], runtime)
        self.mixer = build_part("mixer", spec.parts["mixer"], runtime)
        self.norm2 = build_part("norm", spec.parts["norm2"], runtime)
        self.ffn = build_part("ffn", spec.parts["ffn"], runtime)

    takes_next_norm = True   # forward() accepts the norm part that follows the block

    def children(self):
        return {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "ffn": self.ffn}

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, x, residual, ctx, cache, next_norm=None):
        """``x`` may be None: the previous sub-layer then already added its output into ``residual``.
        Mixers and feed-forwards that set ``fuses_residual`` get the residual and may do the same.
        Those that also set ``emits_normed`` are told which norm reads the residual next
        (``next_norm``: the norm part that follows this block, if any) and may return that norm's
        prepared input; a sub-layer reads such an input only if it sets ``accepts_normed``."""
        y, residual = self.norm1.forward(x, residual)
        a = self._run(self.mixer, y, residual, self.norm2, ctx, cache)
        y, residual = self.norm2.forward(a, residual)
        return self._run(self.ffn, y, residual, next_norm), residual

    @staticmethod
    def _run(part, y, residual, following_norm, *args):
        if hasattr(y, "materialise") and not getattr(part, "accepts_normed", False):
            y = y.materialise()
        kw = {}
        if getattr(part, "fuses_residual", False):
            kw["residual"] = residual
            if getattr(part, "emits_normed", False) and getattr(following_norm, "deferrable", False):
                kw["next_norm"] = (following_norm.weight, following_norm.eps)
        return part.forward(y, *args, **kw)
