"""Arrangements of a block's parts around the residual stream.

``pre_norm``:  x += mixer(norm1(x));  x += feed_forward(norm2(x)); a norm whose consumer can fold it into
its first matrix product is handed over unevaluated (``norm.DeferredNorm``)
(berniehans/titan: engine/engine-core/src/forward_cpu.rs:281-386).  The
residual stream ``x`` is float32 and is updated in place: mixer and
feed-forward add into it in the epilogue of their last matrix product.
"""
from __future__ import annotations

from typing import List

import torch

from ..weights.loader import WeightSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Part


class PreNormBlock(Part):
    def __init__(self, spec):
        if spec.feed_forward is None or spec.mixer_norm is None or spec.feed_forward_norm is None or spec.norms:
            raise ValueError("the pre_norm arrangement takes a mixer, a feed-forward and exactly the two norms before them")
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def weight_specs(self, prefix: str = "") -> List[WeightSpec]:
        out: List[WeightSpec] = []
        for part in self.parts():
            out += part.weight_specs(self.spec.prefix)
        return out

    def bind(self, get) -> None:
        for part in self.parts():
            part.bind(lambda name: get(self.spec.prefix + name))

    @staticmethod
    def _normed(norm, consumer, x, ctx):
        """The norm's rows for the part that consumes them; not yet computed (a DeferredNorm) if the norm can be
        deferred and the part can fold it into its first product."""
        # up to 16 rows: measured after 2,048-token prompts, folding gains 3 % of the step at 12 and 16 sequences and
        # loses 1 to 3 % at 20 to 32 (the kernels take up to 32 rows: twice the float32 rows per weight tile through L2)
        if (getattr(consumer, "folds_norm", False) and hasattr(norm, "deferred") and ctx.options.get("fold_norms", True)
                and x.shape[0] <= int(ctx.options.get("fold_norms_rows", 16))):
            return norm.deferred(x, ctx)
        return norm.forward(x, ctx)

    def forward(self, x: torch.Tensor, ctx, cache) -> None:
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, x, ctx), ctx, cache, x)
        self.feed_forward.forward(self._normed(self.feed_forward_norm, self.feed_forward, x, ctx), ctx, x)


BLOCKS.register("pre_norm", PreNormBlock)
