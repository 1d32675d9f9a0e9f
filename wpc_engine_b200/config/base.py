"""What every architecture's configuration has in common: how a `config.json` is read into
a typed, frozen dataclass, and the error type for a bad one.

An architecture's configuration class lists its own `config.json` keys as dataclass fields
(required ones without a default).  Unknown keys are ignored, as the reference does
(wpc-runtime/src/config.rs:162-168); a missing required key or a value that breaks a rule of
the architecture is a `ConfigError` that names the key.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict


class ConfigError(ValueError):
    """A config.json that cannot describe a model of the architecture it names."""


def read_config_json(path_or_dir: str) -> Dict[str, Any]:
    path = path_or_dir
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return raw


def from_keys(cls, raw: Dict[str, Any]):
    """Builds dataclass `cls` from the keys of `raw` that are its fields."""
    kwargs = {}
    missing = []
    for f in dataclasses.fields(cls):
        if f.name in raw and raw[f.name] is not None:
            kwargs[f.name] = raw[f.name]
        elif f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING:
            missing.append(f.name)
    if missing:
        raise ConfigError(f"{cls.__name__}: config.json lacks required key(s): {', '.join(missing)}")
    return cls(**kwargs)


def require(cond: bool, message: str) -> None:
    if not cond:
        raise ConfigError(message)


def require_int(name: str, value: Any, minimum: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"{name} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"{name} must be >= {minimum}, got {value}")
    return value


def require_number(name: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{name} must be a number, got {value!r}")
    return float(value)
