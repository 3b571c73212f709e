"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, float32 inside, weight used as stored.

berniehans/titan: engine/engine-core/src/forward_cpu.rs:189-200 (eps inside the
sqrt; no ``1 + w``); kernel engine/engine-cuda/kernels/norm_rope.cu:37-80.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels as K
from ..weights.loader import WeightSpec
from .base import NORMS, Norm


class DeferredNorm:
    """An RMS norm that has not run yet: the float32 rows, the norm's weight and eps.  A part that says
    ``folds_norm = True`` may be handed one instead of normalised rows; its first matrix product then takes the
    norm in (the kernel scales by the weight on the way in and by the rows' 1/sqrt(mean(x^2) + eps) on the way
    out), or the part calls ``materialize()`` and goes on as with any tensor."""

    def __init__(self, norm: "RMSNorm", x: torch.Tensor, ctx):
        self.norm, self.x, self.ctx = norm, x, ctx
        self.weight, self.eps = norm.weight, norm.spec.eps
        self.shape, self.dtype = x.shape, ctx.dtype

    def materialize(self) -> torch.Tensor:
        return self.norm.forward(self.x, self.ctx)


def rows_of(h):
    """The normalised rows of ``h``: ``h`` itself, or a deferred norm run now."""
    return h.materialize() if isinstance(h, DeferredNorm) else h


class RMSNorm(Norm):
    def __init__(self, spec):
        self.spec = spec
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        return [WeightSpec(prefix + self.spec.weight, (self.spec.size,), "vector", ("one_plus_normal", 0.1))]

    def bind(self, get) -> None:
        self.weight = get(self.spec.weight)

    def deferred(self, x: torch.Tensor, ctx) -> DeferredNorm:
        return DeferredNorm(self, x, ctx)

    def forward(self, x: torch.Tensor, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        y = ctx.empty((n, self.spec.size))
        K.rmsnorm(x, self.weight, y, self.spec.eps, ctx.stream, rows)
        return y


NORMS.register("rmsnorm", RMSNorm)
