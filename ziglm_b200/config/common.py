"""What every architecture's configuration class needs: the error type, reading config.json, typed getters.

The reference reads config.json with ad-hoc ``if (obj.get(key)) |v|`` tests and
falls back to defaults without saying so (src/safetensors.zig:548-591); here a
key of the wrong kind or out of range is an error that names the key.  These
helpers belong to no architecture: a new configuration class imports them from
here.
"""
from __future__ import annotations

import json
import math
import os
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple


class ConfigError(ValueError):
    """config.json is missing a key, or a value is of the wrong kind or out of range."""


def need_int(d: Mapping[str, Any], key: str, default: Optional[int] = None, minimum: int = 1) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: '{key}' must be an integer, found {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, found {v}")
    return v


def need_float(d: Mapping[str, Any], key: str, default: Optional[float] = None) -> float:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, found {v!r}")
    v = float(v)
    if not math.isfinite(v) or v <= 0.0:
        raise ConfigError(f"config.json: '{key}' must be a positive finite number, found {v}")
    return v


def need_bool(d: Mapping[str, Any], key: str, default: bool) -> bool:
    v = d.get(key, default)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"config.json: '{key}' must be true or false, found {v!r}")
    return v


def need_floats(d: Mapping[str, Any], key: str, length: Optional[int] = None) -> Tuple[float, ...]:
    """A list of positive finite numbers (of ``length`` entries if given)."""
    v = d.get(key)
    if not isinstance(v, (list, tuple)) or not v:
        raise ConfigError(f"config.json: '{key}' must be a non-empty list of numbers, found {v!r}")
    out = []
    for x in v:
        if isinstance(x, bool) or not isinstance(x, (int, float)) or not math.isfinite(float(x)) or float(x) <= 0.0:
            raise ConfigError(f"config.json: '{key}' must hold positive finite numbers, found {x!r}")
        out.append(float(x))
    if length is not None and len(out) != length:
        raise ConfigError(f"config.json: '{key}' must hold {length} numbers, found {len(out)}")
    return tuple(out)


def token_ids(d: Mapping[str, Any], key: str) -> Tuple[int, ...]:
    """A token id or a list of them (the stop set of a checkpoint is written either way)."""
    v = d.get(key)
    if v is None:
        return ()
    items: Sequence[Any] = v if isinstance(v, (list, tuple)) else [v]
    out = []
    for t in items:
        if isinstance(t, bool) or not isinstance(t, int) or t < 0:
            raise ConfigError(f"config.json: '{key}' must be a token id or a list of them, found {v!r}")
        out.append(t)
    return tuple(out)


def architecture_name(d: Any) -> str:
    """``architectures[0]`` of a config.json dictionary: the key of the registry."""
    arch = d.get("architectures") if isinstance(d, Mapping) else None
    if not (isinstance(arch, (list, tuple)) and arch and isinstance(arch[0], str)):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return arch[0]


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path} does not exist") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d
