from .batch import StepContext, StepEntry, StepLayout
from .engine import Engine, EngineOptions, StepError
from .generate import GenerationRequest, GenerationResult, generate
from .model import DecoderModel

__all__ = ["StepContext", "StepEntry", "StepLayout", "Engine", "EngineOptions", "StepError", "GenerationRequest",
           "GenerationResult", "generate", "DecoderModel"]
