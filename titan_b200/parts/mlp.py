"""Gated MLP as a feed-forward: down(act(gate(x)) * up(x)), added into the residual stream.

berniehans/titan: engine/engine-core/src/forward_cpu.rs:369-386 with
silu(g) = g / (1 + exp(-g)) (:210-219); its kernels fuse gate, up and SwiGLU in
one launch (engine/engine-cuda/kernels/gemm_quant.cu:2589).  Here the gate and
up matrices are interleaved row by row at bind time ([2F, H]: gate_0, up_0,
gate_1, ...), so that one matrix product has both halves of every pair in the
same tile and applies the activation in its epilogue.
"""
from __future__ import annotations

from typing import List

import torch

from ..weights.loader import WeightSpec
from . import linear
from .base import FEED_FORWARDS, FeedForward


class GatedMLP(FeedForward):
    def __init__(self, spec):
        if spec.activation != "silu":
            raise ValueError(f"activation '{spec.activation}' is not supported (only 'silu')")
        if spec.intermediate_size <= 0:
            raise ValueError("intermediate_size must be positive")
        self.spec = spec
        self.w_gate_up = self.w_down = None

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p = self.spec, prefix + self.spec.prefix
        return [WeightSpec(p + "gate_proj.weight", (s.intermediate_size, s.hidden_size)),
                WeightSpec(p + "up_proj.weight", (s.intermediate_size, s.hidden_size)),
                WeightSpec(p + "down_proj.weight", (s.hidden_size, s.intermediate_size))]

    def bind(self, get) -> None:
        p = self.spec.prefix
        gate, up = get(p + "gate_proj.weight"), get(p + "up_proj.weight")
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.spec.intermediate_size, self.spec.hidden_size).contiguous()
        del gate, up
        self.w_down = get(p + "down_proj.weight")

    def forward(self, h: torch.Tensor, ctx, out: torch.Tensor) -> None:
        act = ctx.empty((h.shape[0], self.spec.intermediate_size))
        linear.matmul(h, self.w_gate_up, act, linear.EPI_SWIGLU, ctx)
        linear.matmul(act, self.w_down, out, linear.EPI_ADD, ctx)


FEED_FORWARDS.register("gated_mlp", GatedMLP)
