"""Architecture-neutral description of a decoder: what every part is built from.

An architecture's typed configuration (for instance ``Qwen3Config``) turns its
own ``config.json`` keys into a ``ModelSpec``.  Parts are built from the specs
below and never see the architecture's configuration, so no part knows which
model it is in.  A spec carries a ``kind`` string that names the part's class in
the part registries (``titan_b200.parts``), its sizes and its constants.

berniehans/titan keeps the same numbers in one flat ``ModelConfig``
(engine/engine-io/src/config.rs:36-72) and hard-codes the arrangement in
``ForwardDriver`` (engine/engine-core/src/forward_driver.rs:988-1207); here the
arrangement is data.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that is missing a key, or holds a value that is not supported."""


@dataclass(frozen=True)
class NormSpec:
    kind: str                 # "rmsnorm"
    size: int
    eps: float
    weight: str               # tensor name relative to the owner's prefix


@dataclass(frozen=True)
class PositionSpec:
    kind: str                 # "rope" | "none"
    rotary_dim: int = 0       # leading dims of a head that are rotated
    theta: float = 10000.0
    pairing: str = "half"     # (k, k + rotary_dim/2)


@dataclass(frozen=True)
class MixerSpec:
    kind: str                 # "attention"
    hidden_size: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None          # None: all keys; n: keys p-n < t <= p
    qk_norm: Optional[NormSpec] = None    # per-head norm on Q and K before the rotation
    position: PositionSpec = PositionSpec("none")
    softmax_scale: Optional[float] = None  # None: 1/sqrt(head_dim)
    cache_from: Optional[int] = None      # read (and do not write) this layer's cache
    prefix: str = "self_attn."
    extra: Tuple[Tuple[str, Any], ...] = ()   # for mixers defined outside the package

    def option(self, key: str, default: Any = None) -> Any:
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                 # "gated_mlp"
    hidden_size: int
    intermediate_size: int = 0
    activation: str = "silu"
    prefix: str = "mlp."
    extra: Tuple[Tuple[str, Any], ...] = ()

    def option(self, key: str, default: Any = None) -> Any:
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One block: which mixer, which feed-forward, which norms, how arranged."""
    index: int
    arrangement: str          # "pre_norm"
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    prefix: str               # "model.layers.3."


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    order: Tuple[int, ...]                # indices into ``layers`` in running order
    final_norm: NormSpec
    embedding: str = "model.embed_tokens.weight"
    lm_head: Optional[str] = "lm_head.weight"   # None: tied to the embedding
    max_positions: int = 4096
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i in self.order:
            if not 0 <= i < len(self.layers):
                raise ConfigError(f"layer order names layer {i}, but there are {len(self.layers)} layers")
        for layer in self.layers:
            src = layer.mixer.cache_from
            if src is not None:
                if not 0 <= src < len(self.layers) or self.layers[src].mixer.cache_from is not None:
                    raise ConfigError(f"layer {layer.index} reads the cache of layer {src}, which owns none")
                if src not in self.order or self.order.index(src) > self.order.index(layer.index):
                    raise ConfigError(f"layer {layer.index} reads the cache of layer {src} before it is written")
