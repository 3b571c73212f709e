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


class RMSNorm(Norm):
    def __init__(self, spec):
        self.spec = spec
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        return [WeightSpec(prefix + self.spec.weight, (self.spec.size,), "vector", ("one_plus_normal", 0.1))]

    def bind(self, get) -> None:
        self.weight = get(self.spec.weight)

    def forward(self, x: torch.Tensor, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.numel()
        y = ctx.empty((n, self.spec.size))
        K.rmsnorm(x, self.weight, y, self.spec.eps, ctx.stream, rows)
        return y


NORMS.register("rmsnorm", RMSNorm)
