"""Typed configuration of the Qwen3 dense architecture, from its config.json keys.

berniehans/titan reads the same quantities from GGUF metadata
(engine/engine-io/src/config.rs:76-177): block_count, embedding_length,
feed_forward_length, attention.head_count, attention.head_count_kv (default:
heads, :115), attention.key_length (default hidden/heads, :119-120),
context_length (default 4096, :116), rope.freq_base (default 10000, :29),
attention.layer_norm_rms_epsilon (default 1e-5, :31), eos token (:145-148).
A missing required key is an error that names the key (:94).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .spec import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)

_REQUIRED = ("num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads", "vocab_size")


def _as_int(d: Dict[str, Any], key: str, default: Optional[int] = None) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json lacks the key '{key}'")
    if isinstance(v, bool) or (isinstance(v, float) and v != int(v)) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json key '{key}' must be an integer, found {v!r}")
    v = int(v)
    if v <= 0:
        raise ConfigError(f"config.json key '{key}' must be positive, found {v}")
    return v


@dataclass(frozen=True)
class Qwen3Config:
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    layer_windows: Tuple[Optional[int], ...]      # per layer: None = all keys
    eos_token_ids: Tuple[int, ...]
    hidden_act: str = "silu"
    architecture: str = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ #
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen3Config":
        for key in _REQUIRED:
            if key not in d:
                raise ConfigError(f"config.json lacks the key '{key}'")
        layers = _as_int(d, "num_hidden_layers")
        hidden = _as_int(d, "hidden_size")
        heads = _as_int(d, "num_attention_heads")
        kv_heads = _as_int(d, "num_key_value_heads", heads)
        if d.get("head_dim") is None:
            if hidden % heads:
                raise ConfigError(f"no 'head_dim', and hidden_size {hidden} is not a multiple of {heads} heads")
            head_dim = hidden // heads
        else:
            head_dim = _as_int(d, "head_dim")
        if heads % kv_heads:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be even for the rotary pairing")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act '{act}' is not supported (only 'silu')")
        if d.get("attention_bias"):
            raise ConfigError("attention_bias = true is not supported")
        if d.get("mlp_bias"):
            raise ConfigError("mlp_bias = true is not supported")
        if d.get("partial_rotary_factor") not in (None, 1, 1.0):
            raise ConfigError("partial_rotary_factor other than 1 is not supported")
        theta = d.get("rope_theta")
        # the frequency base and a scaling rule travel either as rope_theta + rope_scaling or, in newer
        # files, together in rope_parameters; only the unscaled ("default") rule is built
        for key in ("rope_scaling", "rope_parameters"):
            rule = d.get(key)
            if rule in (None, {}):
                continue
            if not isinstance(rule, dict):
                raise ConfigError(f"config.json key '{key}' must be an object, found {rule!r}")
            kind = rule.get("rope_type", rule.get("type", "default"))
            if kind != "default" or any(k not in ("rope_type", "type", "rope_theta") for k in rule):
                raise ConfigError(f"{key} {rule!r} is not supported (only the unscaled rotary encoding)")
            if rule.get("rope_theta") is not None:
                if theta is not None and float(theta) != float(rule["rope_theta"]):
                    raise ConfigError(f"rope_theta {theta} and {key}.rope_theta {rule['rope_theta']} disagree")
                theta = rule["rope_theta"]
        eps = float(d.get("rms_norm_eps", 1e-5))
        theta = float(10000.0 if theta is None else theta)
        if not eps > 0 or not theta > 0:
            raise ConfigError("rms_norm_eps and rope_theta must be positive")
        vocab = _as_int(d, "vocab_size")

        window = d.get("sliding_window")
        types = d.get("layer_types")
        if types is not None:
            if len(types) != layers:
                raise ConfigError(f"layer_types has {len(types)} entries for {layers} layers")
            for t in types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"layer type '{t}' is not known (full_attention, sliding_attention)")
            if "sliding_attention" in types and window is None:
                raise ConfigError("layer_types names sliding_attention but sliding_window is null")
            windows = tuple(_as_int(d, "sliding_window") if t == "sliding_attention" else None for t in types)
        elif d.get("use_sliding_window") and window is not None:
            first = int(d.get("max_window_layers", layers))
            windows = tuple(_as_int(d, "sliding_window") if i >= first else None for i in range(layers))
        else:
            windows = (None,) * layers

        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]))
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"eos_token_id {e} lies outside the vocabulary of {vocab}")
        return cls(
            num_hidden_layers=layers, hidden_size=hidden, intermediate_size=_as_int(d, "intermediate_size"),
            num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, vocab_size=vocab,
            rms_norm_eps=eps, rope_theta=theta,
            max_position_embeddings=_as_int(d, "max_position_embeddings", 4096),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            layer_windows=windows, eos_token_ids=eos_ids, hidden_act=act,
            architecture=(d.get("architectures") or ["Qwen3ForCausalLM"])[0])

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        d: Dict[str, Any] = {
            "architectures": [self.architecture], "model_type": "qwen3",
            "num_hidden_layers": self.num_hidden_layers, "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "vocab_size": self.vocab_size, "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": self.hidden_act,
            "attention_bias": False, "rope_scaling": None,
        }
        wins = [w for w in self.layer_windows if w is not None]
        if wins:
            d["sliding_window"] = wins[0]
            d["layer_types"] = ["sliding_attention" if w is not None else "full_attention" for w in self.layer_windows]
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    # ------------------------------------------------------------------ #
    def to_model_spec(self) -> ModelSpec:
        """Pre-norm blocks of GQA attention (per-head RMSNorm on Q and K, rotary
        over the whole head) and a SiLU-gated MLP; final RMSNorm; LM head tied or
        not (engine/engine-core/src/forward_cpu.rs:281-395)."""
        wins = set(w for w in self.layer_windows if w is not None)
        if len(wins) > 1:
            raise ConfigError("one sliding_window per model")
        H, hd, eps = self.hidden_size, self.head_dim, self.rms_norm_eps
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = MixerSpec(
                kind="attention", hidden_size=H, num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads, head_dim=hd, window=self.layer_windows[i],
                qk_norm=NormSpec("rmsnorm", hd, eps, "{}_norm.weight"),
                position=PositionSpec("rope", rotary_dim=hd, theta=self.rope_theta, pairing="half"))
            ffn = FeedForwardSpec(kind="gated_mlp", hidden_size=H, intermediate_size=self.intermediate_size,
                                  activation=self.hidden_act)
            layers.append(LayerSpec(
                index=i, arrangement="pre_norm", mixer=mixer, feed_forward=ffn,
                mixer_norm=NormSpec("rmsnorm", H, eps, "input_layernorm.weight"),
                feed_forward_norm=NormSpec("rmsnorm", H, eps, "post_attention_layernorm.weight"),
                prefix=f"model.layers.{i}."))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=H, vocab_size=self.vocab_size, layers=tuple(layers),
            order=tuple(range(self.num_hidden_layers)),
            final_norm=NormSpec("rmsnorm", H, eps, "model.norm.weight"),
            lm_head=None if self.tie_word_embeddings else "lm_head.weight",
            max_positions=self.max_position_embeddings, stop_token_ids=self.eos_token_ids)
        spec.validate()
        return spec
