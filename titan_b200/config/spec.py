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


def _lookup(pairs, key, default):
    for k, v in pairs:
        if k == key:
            return v
    return default


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
    # Tensor names by role, relative to ``prefix``; roles a part knows and that are not listed keep the
    # part's default.  Attention: "q", "k", "v", "o" (defaults q_proj.weight ...), or "qkv" for a checkpoint
    # that stores the three projections as one [Q + 2 KV, H] tensor.
    names: Tuple[Tuple[str, str], ...] = ()
    extra: Tuple[Tuple[str, Any], ...] = ()   # for mixers defined outside the package

    def option(self, key: str, default: Any = None) -> Any:
        return _lookup(self.extra, key, default)

    def name(self, role: str, default: Optional[str] = None) -> Optional[str]:
        return _lookup(self.names, role, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                 # "gated_mlp"
    hidden_size: int
    intermediate_size: int = 0
    activation: str = "silu"
    prefix: str = "mlp."
    # Tensor names by role: "gate", "up", "down" (defaults gate_proj.weight ...), or "gate_up" for a
    # checkpoint that stores gate and up as one [2 F, H] tensor (gate rows first).
    names: Tuple[Tuple[str, str], ...] = ()
    extra: Tuple[Tuple[str, Any], ...] = ()

    def option(self, key: str, default: Any = None) -> Any:
        return _lookup(self.extra, key, default)

    def name(self, role: str, default: Optional[str] = None) -> Optional[str]:
        return _lookup(self.names, role, default)


@dataclass(frozen=True)
class LayerSpec:
    """One block: which mixer, which feed-forward, which norms, how arranged.  The arrangement gives the
    fields their meaning: ``pre_norm`` needs all four parts; another arrangement may do without a
    feed-forward (None), or take more norms than two from ``norms`` (a norm after each part as well as
    before it, say) and its own constants from ``extra``."""
    index: int
    arrangement: str          # "pre_norm"
    mixer: MixerSpec
    feed_forward: Optional[FeedForwardSpec]
    mixer_norm: Optional[NormSpec]
    feed_forward_norm: Optional[NormSpec]
    prefix: str               # "model.layers.3."
    norms: Tuple[NormSpec, ...] = ()          # further norms, in the order the arrangement defines
    extra: Tuple[Tuple[str, Any], ...] = ()

    def option(self, key: str, default: Any = None) -> Any:
        return _lookup(self.extra, key, default)


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
    embedding_scale: Optional[float] = None   # the embedded rows are multiplied by this (None: as stored)
    logit_scale: Optional[float] = None       # the logits are multiplied by this (None: as computed)

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i in self.order:
            if not 0 <= i < len(self.layers):
                raise ConfigError(f"layer order names layer {i}, but there are {len(self.layers)} layers")
        for layer in self.layers:
            src = layer.mixer.cache_from
            if src is None:
                continue
            me = layer.mixer
            if not 0 <= src < len(self.layers) or self.layers[src].mixer.cache_from is not None:
                raise ConfigError(f"layer {layer.index} reads the cache of layer {src}, which owns none")
            if layer.index not in self.order:
                raise ConfigError(f"layer {layer.index} reads the cache of layer {src} but never runs (it is not in the order)")
            if src not in self.order or self.order.index(src) > self.order.index(layer.index):
                raise ConfigError(f"layer {layer.index} reads the cache of layer {src} before it is written")
            owner = self.layers[src].mixer
            if owner.kind != me.kind:
                raise ConfigError(f"layer {layer.index} ({me.kind}) reads the cache of layer {src}, whose mixer is of another kind ({owner.kind})")
            if owner.window != me.window:
                raise ConfigError(f"layer {layer.index} reads the cache of layer {src}, which keeps a window of {owner.window} keys, "
                                  f"with a window of {me.window}: a reader must see exactly what the owner keeps")
            if owner.head_dim != me.head_dim:
                raise ConfigError(f"layer {layer.index} has heads of {me.head_dim}, the cache of layer {src} holds heads of {owner.head_dim}")
            if owner.num_kv_heads <= 0 or me.num_heads % owner.num_kv_heads:
                raise ConfigError(f"layer {layer.index} has {me.num_heads} query heads, not a multiple of the {owner.num_kv_heads} "
                                  f"kv heads in the cache of layer {src}")
