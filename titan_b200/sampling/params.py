"""Sampling options, with berniehans/titan's names, meanings and defaults
(engine/engine-core/src/sampler.rs:13-54): temperature 0.7 (<= 1e-4 is greedy), top_p 0.9,
top_k 40 (0 disables), repetition_penalty 1.1 (1.0 disables), seed None (42 is used,
engine/engine-server/src/server.rs:252); ``SamplerParams.greedy()`` is its greedy preset.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

GREEDY_TEMPERATURE = 1e-4
DEFAULT_SEED = 42


@dataclass(frozen=True)
class SamplerParams:
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 40
    repetition_penalty: float = 1.1
    seed: Optional[int] = None

    @classmethod
    def greedy(cls) -> "SamplerParams":
        return cls(temperature=0.0, top_p=1.0, top_k=0, repetition_penalty=1.0, seed=None)

    def is_greedy(self) -> bool:
        return self.temperature <= GREEDY_TEMPERATURE

    def validate(self) -> None:
        if not (self.temperature >= 0.0):
            raise ValueError(f"temperature must be >= 0, found {self.temperature}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must lie in (0, 1], found {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, found {self.top_k}")
        if not (self.repetition_penalty >= 1.0):
            raise ValueError(f"repetition_penalty must be >= 1, found {self.repetition_penalty}")

    def seed_value(self) -> int:
        return (DEFAULT_SEED if self.seed is None else int(self.seed)) & ((1 << 63) - 1)
