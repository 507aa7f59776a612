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

    def children(self):
        return {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "ffn": self.ffn}

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, x, residual, ctx, cache):
        """``x`` may be None: the previous sub-layer then already added its output into ``residual``.
        Mixers and feed-forwards that set ``fuses_residual`` get the residual and may do the same."""
        y, residual = self.norm1.forward(x, residual)
        if getattr(self.mixer, "fuses_residual", False):
            a = self.mixer.forward(y, ctx, cache, residual=residual)
        else:
            a = self.mixer.forward(y, ctx, cache)
        y, residual = self.norm2.forward(a, residual)
        if getattr(self.ffn, "fuses_residual", False):
            return self.ffn.forward(y, residual=residual), residual
        return self.ffn.forward(y), residual
