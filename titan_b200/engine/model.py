"""A decoder assembled from a ``ModelSpec``: embedding, blocks in their running order,
final norm and LM head.

The running order is data (``ModelSpec.order``): it may name a layer twice, and
a layer's mixer may read another layer's cache (``MixerSpec.cache_from``).
berniehans/titan hard-codes ``for layer in 0..L`` (engine/engine-core/src/
forward_driver.rs:988, 2149-2334) and computes logits for the last position
only (:1215-1238); here the wanted rows are gathered before the final norm, so
the LM head runs on those rows alone.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed
from ..parts import NORMS, build_block, declare_weights, linear
from ..weights.loader import WeightSource, WeightSpec


class DecoderModel:
    def __init__(self, spec):
        spec.validate()
        self.spec = spec
        self.blocks = [build_block(layer) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None

    def declared_weights(self) -> List[WeightSpec]:
        return declare_weights(self.spec)

    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """One entry per RUN of the order, so a layer that runs twice keeps two caches."""
        return [self.blocks[i].mixer.cache_need() for i in self.spec.order]

    def cache_run_of(self, run: int) -> int:
        """The run whose cache the ``run``-th block of the order uses."""
        src = self.spec.layers[self.spec.order[run]].mixer.cache_from
        return run if src is None else self.spec.order.index(src)

    def load(self, source: WeightSource) -> None:
        by_name = {w.name: w for w in self.declared_weights()}
        get = lambda name: source.get(by_name[name])
        self.embedding = get(self.spec.embedding)
        for b in self.blocks:
            b.bind(get)
        self.final_norm.bind(get)
        self.lm_head = self.embedding if self.spec.lm_head is None else get(self.spec.lm_head)

    def weight_bytes(self) -> int:
        """Bytes a decode step reads: every matrix once (the embedding table only as LM head when tied)."""
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        for i in set(self.spec.order):
            for part in self.blocks[i].parts():
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        add(v)
        add(self.lm_head)
        add(self.final_norm.weight)
        return total

    # ------------------------------------------------------------------ #
    def forward_hidden(self, ctx, cache) -> torch.Tensor:
        """The residual stream [T, H] (float32) after the last block."""
        lay = ctx.layout
        x = torch.empty((lay.T, self.spec.hidden_size), dtype=torch.float32, device=ctx.device)
        K.embed(self.embedding, lay.tokens, x, ctx.stream)
        if self.spec.embedding_scale is not None:
            K.scale_f32(x, float(self.spec.embedding_scale), ctx.stream)
        if "row_sums" not in ctx.scratch:      # places where folded norms leave sums of squares: one per run of a layer
            ctx.scratch["row_sums"] = torch.zeros((len(self.spec.order), 16, 32), dtype=torch.float32, device=ctx.device)
        for run, i in enumerate(self.spec.order):
            self.blocks[i].forward(x, ctx, cache.view_for_layer(self.cache_run_of(run)))
        return x

    def logits(self, x: torch.Tensor, ctx, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] at the given rows of the residual stream."""
        hn = self.final_norm.forward(x, ctx, rows)
        out = torch.empty((rows.numel(), self.spec.vocab_size), dtype=torch.float32, device=ctx.device)
        linear.matmul(hn, self.lm_head, out, linear.EPI_F32, ctx)
        if self.spec.logit_scale is not None:
            K.scale_f32(out, float(self.spec.logit_scale), ctx.stream)
        return out
