"""Gated MLP as a feed-forward: down(act(gate(x)) * up(x)), added into the residual stream.

berniehans/titan: engine/engine-core/src/forward_cpu.rs:369-386 with
silu(g) = g / (1 + exp(-g)) (:210-219); its kernels fuse gate, up and SwiGLU in
one launch (engine/engine-cuda/kernels/gemm_quant.cu:2589).  Here the gate and
up matrices are interleaved row by row at bind time ([2F, H]: gate_0, up_0,
gate_1, ...), so that one matrix product has both halves of every pair in the
same tile and applies the activation in its epilogue.  The tensors' names come
from the spec (``FeedForwardSpec.names``): gate_proj / up_proj / down_proj
``.weight`` by default, or one stored [2F, H] tensor (gate rows, then up rows)
under the role "gate_up".
"""
from __future__ import annotations

from typing import List

import torch

from ..weights.loader import WeightSpec
from .. import kernels as K
from . import linear
from .base import FEED_FORWARDS, FeedForward
from .norm import DeferredNorm, rows_of


class GatedMLP(FeedForward):
    folds_norm = True           # a decode step's gate-and-up product takes the norm before it in

    def __init__(self, spec):
        if spec.activation != "silu":
            raise ValueError(f"activation '{spec.activation}' is not supported (only 'silu')")
        if spec.intermediate_size <= 0:
            raise ValueError("intermediate_size must be positive")
        self.spec = spec
        self.w_gate_up = self.w_down = None

    def _names(self):
        s = self.spec
        names = {role: s.name(role, role + "_proj.weight") for role in ("gate", "up", "down")}
        names["gate_up"] = s.name("gate_up")
        return names

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        s, p, n = self.spec, prefix + self.spec.prefix, self._names()
        if n["gate_up"] is not None:
            first = [WeightSpec(p + n["gate_up"], (2 * s.intermediate_size, s.hidden_size))]
        else:
            first = [WeightSpec(p + n["gate"], (s.intermediate_size, s.hidden_size)),
                     WeightSpec(p + n["up"], (s.intermediate_size, s.hidden_size))]
        return first + [WeightSpec(p + n["down"], (s.hidden_size, s.intermediate_size))]

    def bind(self, get) -> None:
        p, n, F = self.spec.prefix, self._names(), self.spec.intermediate_size
        if n["gate_up"] is not None:
            both = get(p + n["gate_up"])
            gate, up = both[:F], both[F:]
        else:
            gate, up = get(p + n["gate"]), get(p + n["up"])
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * F, self.spec.hidden_size).contiguous()
        del gate, up
        self.w_down = get(p + n["down"])

    def forward(self, h, ctx, out: torch.Tensor) -> None:
        act = ctx.empty((h.shape[0], self.spec.intermediate_size))
        if (isinstance(h, DeferredNorm) and ctx.options.get("gemm", "fast") != "plain" and self.w_gate_up.dtype == torch.bfloat16
                and K.gemm_tc_normed_accepts(h.x, h.weight, self.w_gate_up, act, linear.EPI_SWIGLU, None)):
            K.gemm_tc_normed(h.x, h.weight, h.eps, self.w_gate_up, act, linear.EPI_SWIGLU, ctx.stream)
        else:
            linear.matmul(rows_of(h), self.w_gate_up, act, linear.EPI_SWIGLU, ctx)
        linear.matmul(act, self.w_down, out, linear.EPI_ADD, ctx)


FEED_FORWARDS.register("gated_mlp", GatedMLP)
