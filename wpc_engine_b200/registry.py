"""One registry from an architecture's name to its configuration class and model builder.

The name is `architectures[0]` of config.json, or `model_type` where that list is absent.
An unknown name is an error: nothing falls back to another architecture (the reference's
`--arch auto` treats every unknown model_type as Qwen2, wpc-runtime/src/main.rs:74-78; here
that would hide a wrong model folder).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple

from .config.base import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build: Callable[[Any], Any]
    model_types: Tuple[str, ...] = ()


_ARCHITECTURES: Dict[str, Architecture] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_class: type, build: Callable[[Any], Any],
                          model_types: Tuple[str, ...] = (), replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name} is registered already")
    _ARCHITECTURES[name] = Architecture(name, config_class, build, tuple(model_types))
    for mt in model_types:
        _MODEL_TYPES[mt] = name


def unregister_architecture(name: str) -> None:
    arch = _ARCHITECTURES.pop(name)
    for mt in arch.model_types:
        _MODEL_TYPES.pop(mt, None)


def architecture_names():
    return sorted(_ARCHITECTURES)


def resolve(raw: Dict[str, Any]) -> Architecture:
    """The registered architecture that a config.json (as a dict) names."""
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    if names:
        if names[0] in _ARCHITECTURES:
            return _ARCHITECTURES[names[0]]
        raise ConfigError(f"unknown architecture {names[0]!r}; registered: {architecture_names()}")
    mt = raw.get("model_type")
    if mt in _MODEL_TYPES:
        return _ARCHITECTURES[_MODEL_TYPES[mt]]
    raise ConfigError(f"config.json names no known architecture (architectures={names!r}, "
                      f"model_type={mt!r}); registered: {architecture_names()}")


def config_from_folder(folder: str):
    raw = read_config_json(folder)
    arch = resolve(raw)
    return arch, arch.config_class.from_dict(raw)


def _register_builtin() -> None:
    from .config.qwen2 import Qwen2Config
    from .models.qwen2 import build_qwen2
    register_architecture(Qwen2Config.ARCHITECTURE, Qwen2Config, build_qwen2, model_types=("qwen2",))


_register_builtin()
