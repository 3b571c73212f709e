"""titan_b200: a small, whole text-generation library for one NVIDIA B200.

Everything between a request's token ids and its next token for the Qwen3 dense
architecture, on hand-written sm_100a kernels:

    from titan_b200 import Engine, SamplerParams
    engine = Engine.from_pretrained("model_dir", dtype="bfloat16", max_tokens=65536)
    results = engine.generate([[1, 2, 3], [4, 5]], max_tokens=32, params=SamplerParams.greedy())
"""
from .config import ConfigError, Qwen3Config, load_config, register_architecture
from .engine import Engine, EngineOptions, GenerationRequest, GenerationResult, StepEntry, StepError
from .sampling import SamplerParams
from .weights import WeightError, write_model_folder

__version__ = "0.1.0"
__all__ = ["ConfigError", "Qwen3Config", "load_config", "register_architecture", "Engine", "EngineOptions",
           "GenerationRequest", "GenerationResult", "StepEntry", "StepError", "SamplerParams", "WeightError",
           "write_model_folder"]
