"""Interfaces of the parts a decoder is put together from, and their registries.

A part is built from its spec alone (``titan_b200.config.spec``); it declares
the tensors it owns, receives them, and runs on the rows of a step.  It never
sees the model's configuration or the other parts.

Interfaces
----------
Norm            ``forward(x_f32[T,H], ctx, rows=None) -> y[T',H]`` in the compute dtype;
                ``rows`` (int32 on the device) picks rows first.
Mixer           ``cache_need() -> CacheNeed | None`` what it asks of the cache;
                ``forward(h[T,H], ctx, cache, out_f32[T,H])`` adds its result into
                ``out`` (the float32 residual stream).  ``cache`` is ``(group, index)``
                from ``SequenceCache.view_for_layer`` or None.
FeedForward     ``forward(h[T,H], ctx, out_f32[T,H])`` adds its result into ``out``.
PositionEncoding  owned by a mixer; ``kernel_args(device)`` returns the argument block that the
                mixer hands to its kernels without looking inside (``kernels.RotaryArgs``: table of
                inverse frequencies, rotated dims, an offset on positions, a factor on cosines and
                sines).  The default builds it from ``rotary_dim`` and ``tables(device)["inv_freq"]``.
Block           ``forward(x_f32, ctx, cache)`` runs norms, mixer and feed-forward in its arrangement.

All of them: ``weight_specs(prefix) -> [WeightSpec]`` and ``bind(get)``, where
``get(relative_name) -> tensor`` hands out the declared tensors on the device.

Registering a new kind: ``MIXERS.register("name", Class)`` (likewise
FEED_FORWARDS, NORMS, POSITIONS, BLOCKS); the class is constructed as
``Class(spec)``.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from ..cache.groups import CacheNeed
from ..weights.loader import WeightSpec


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._classes: Dict[str, type] = {}

    def register(self, kind: str, cls: type) -> type:
        self._classes[kind] = cls
        return cls

    def build(self, spec):
        if spec.kind not in self._classes:
            raise KeyError(f"no {self.what} of kind '{spec.kind}' is registered; known: {', '.join(sorted(self._classes))}")
        return self._classes[spec.kind](spec)

    def kinds(self) -> List[str]:
        return sorted(self._classes)


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block arrangement")


class Part:
    # Whether a decode step with this part may be captured as a CUDA graph: its forward launches kernels on the
    # step's stream and reads nothing of the device on the host.  A part that cannot promise this says False,
    # and the engine runs every step of a model that holds it eagerly.
    capturable = True

    def weight_specs(self, prefix: str) -> List[WeightSpec]:
        return []

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        pass


class Norm(Part):
    def forward(self, x: torch.Tensor, ctx, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    rotary_dim = 0

    def tables(self, device) -> Dict[str, torch.Tensor]:
        return {}

    def kernel_args(self, device):
        """The block a mixer passes to its kernels.  Plain rotary: the table alone; an encoding with an
        offset on positions or a factor on the rotation overrides this (or sets the two fields)."""
        from .. import kernels as K
        held = getattr(self, "_held_tables", None)
        if held is None:
            held = self._held_tables = self.tables(device)      # kept: the block holds an address into them
        inv = held.get("inv_freq")
        return K.RotaryArgs(None if inv is None else inv.data_ptr(), int(self.rotary_dim) if inv is not None else 0, 0.0, 1.0)


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, h: torch.Tensor, ctx, cache, out: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx, out: torch.Tensor) -> None:
        raise NotImplementedError
