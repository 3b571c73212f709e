"""Position encodings that a mixer applies to its queries and keys.

``rope``: half-split rotary over the first ``rotary_dim`` dims of a head:
for k < rotary_dim/2, angle = position * theta^(-2k/rotary_dim), and the pair
(k, k + rotary_dim/2) is rotated (berniehans/titan:
engine/engine-core/src/forward_cpu.rs:226-241; rotary_dim = head_dim,
forward_driver.rs:608).  The inverse frequencies are computed in float64 on the
host and rounded once to float32; the angle and its sine and cosine are float32
in the kernel.

``none``: no table; the mixer's kernel then leaves the heads as they are.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import POSITIONS, PositionEncoding


class Rotary(PositionEncoding):
    def __init__(self, spec):
        if spec.pairing != "half":
            raise ValueError(f"rotary pairing '{spec.pairing}' is not supported (only 'half')")
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be positive and even")
        self.spec = spec
        self._tables: Dict[str, torch.Tensor] = {}

    @property
    def rotary_dim(self) -> int:
        return self.spec.rotary_dim

    def tables(self, device) -> Dict[str, torch.Tensor]:
        if not self._tables:
            rot = self.spec.rotary_dim
            k = torch.arange(rot // 2, dtype=torch.float64)
            inv = torch.tensor(self.spec.theta, dtype=torch.float64) ** (-2.0 * k / rot)
            self._tables = {"inv_freq": inv.to(torch.float32).to(device)}
        return self._tables


class NoPosition(PositionEncoding):
    def __init__(self, spec):
        self.spec = spec


POSITIONS.register("rope", Rotary)
POSITIONS.register("none", NoPosition)
