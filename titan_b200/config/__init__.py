from .spec import (ConfigError, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)
from .qwen3 import Qwen3Config
from .registry import config_from_dict, known_architectures, load_config, register_architecture

register_architecture("Qwen3ForCausalLM", Qwen3Config)

__all__ = ["ConfigError", "FeedForwardSpec", "LayerSpec", "MixerSpec", "ModelSpec", "NormSpec",
           "PositionSpec", "Qwen3Config", "config_from_dict", "known_architectures", "load_config",
           "register_architecture"]
