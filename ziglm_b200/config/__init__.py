from .llama import ConfigError, LlamaConfig, RopeScaling, read_config_json
from .registry import (config_from_dict, config_from_folder, register_architecture,
                       registered_architectures, unregister_architecture)
from .spec import (FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)

__all__ = [
    "ConfigError", "LlamaConfig", "RopeScaling", "read_config_json",
    "config_from_dict", "config_from_folder", "register_architecture",
    "registered_architectures", "unregister_architecture",
    "FeedForwardSpec", "LayerSpec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec",
]
