"""ziglm_b200: a small generation library for Llama-style decoders on one B200.

The library surface follows the reference's re-exports (src/root.zig:22-35):
``Engine``, ``EngineOptions``, ``GenerationOptions``, ``GenerationStats``,
``SamplerParams`` (the reference's ``Sampler`` options).
"""
from .config import ConfigError, LlamaConfig, config_from_dict, config_from_folder, register_architecture
from .engine import (Engine, EngineOptions, GenerationOptions, GenerationResult, GenerationStats, StepError)
from .sampling import SamplerParams
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "LlamaConfig", "config_from_dict", "config_from_folder", "register_architecture",
           "Engine", "EngineOptions", "GenerationOptions", "GenerationResult", "GenerationStats", "StepError",
           "SamplerParams", "WeightError", "write_random_model"]
__version__ = "0.1.0"
