"""One registry from the architecture name in config.json to its configuration class.

The reference's registry is a substring match from ``architectures[0]`` to an
enum (src/safetensors.zig:517-532, src/types.zig:225-238) whose values the
forward pass then branches on.  Here the name selects a configuration class;
the class turns config.json into a typed configuration and that into a
:class:`~ziglm_b200.config.spec.ModelSpec`, which is all the engine needs.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Mapping

from .common import ConfigError, architecture_name, read_config_json
from .llama import LlamaConfig
from .spec import ModelSpec

_ARCHITECTURES: Dict[str, Any] = {}


def register_architecture(name: str, config_class: Any) -> None:
    """``config_class`` needs ``from_dict(mapping)`` and, on its instances, ``model_spec()``."""
    if name in _ARCHITECTURES and _ARCHITECTURES[name] is not config_class:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = config_class


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_from_dict(d: Mapping[str, Any]):
    arch = architecture_name(d)
    cls = _ARCHITECTURES.get(arch)
    if cls is None:
        raise ConfigError(
            f"architecture {arch!r} is not registered (known: {', '.join(registered_architectures())})")
    return cls.from_dict(d)


def config_from_folder(folder: str):
    """config.json of a model folder.  A generation_config.json beside it supplies ``eos_token_id`` and
    ``bos_token_id`` when config.json has none (checkpoints keep the full stop set there)."""
    d = dict(read_config_json(folder))
    extra = os.path.join(folder, "generation_config.json")
    if os.path.isfile(extra):
        try:
            with open(extra) as f:
                gen = json.load(f)
        except (OSError, ValueError) as e:
            raise ConfigError(f"{extra}: cannot be read as JSON ({e})") from None
        if isinstance(gen, dict):
            for key in ("eos_token_id", "bos_token_id"):
                if d.get(key) is None and gen.get(key) is not None:
                    d[key] = gen[key]
    return config_from_dict(d)


register_architecture(LlamaConfig.ARCHITECTURE, LlamaConfig)
