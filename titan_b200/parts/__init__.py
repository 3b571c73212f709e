"""Parts of a decoder and their registries; importing this package registers the built-in kinds."""
from __future__ import annotations

from typing import List

from ..weights.loader import WeightSpec
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, FeedForward, Mixer, Norm, Part,
                   PositionEncoding, Registry)
from . import attention, block, mlp, norm, rotary  # noqa: F401  (registration)


def build_block(layer_spec):
    kind = layer_spec.arrangement
    if kind not in BLOCKS._classes:
        raise KeyError(f"no block arrangement '{kind}' is registered; known: {', '.join(BLOCKS.kinds())}")
    return BLOCKS._classes[kind](layer_spec)


def declare_weights(model_spec) -> List[WeightSpec]:
    """Every tensor the model owns, in file order, without touching a device."""
    specs = [WeightSpec(model_spec.embedding, (model_spec.vocab_size, model_spec.hidden_size))]
    for layer in model_spec.layers:
        specs += build_block(layer).weight_specs()
    specs += NORMS.build(model_spec.final_norm).weight_specs("")
    if model_spec.lm_head is not None:
        specs.append(WeightSpec(model_spec.lm_head, (model_spec.vocab_size, model_spec.hidden_size)))
    return specs


__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "FeedForward", "Mixer", "Norm", "Part",
           "PositionEncoding", "Registry", "build_block", "declare_weights"]
