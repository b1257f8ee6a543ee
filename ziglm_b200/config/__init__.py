from .common import ConfigError, read_config_json
from .llama import LlamaConfig, RopeScaling
from .registry import (config_from_dict, config_from_folder, register_architecture,
                       registered_architectures, unregister_architecture)
from .shapes import SHAPES, shape
from .spec import (FeedForwardSpec, HookSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)

__all__ = [
    "ConfigError", "LlamaConfig", "SHAPES", "shape", "RopeScaling", "read_config_json",
    "config_from_dict", "config_from_folder", "register_architecture",
    "registered_architectures", "unregister_architecture",
    "FeedForwardSpec", "HookSpec", "LayerSpec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec",
]
