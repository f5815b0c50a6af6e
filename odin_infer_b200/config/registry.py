"""The one registry from an architecture's name (config.json "architectures"[0])
to its configuration class and its model builder.

Adding an architecture is one call of `register_architecture`: a subclass of
ModelConfig that reads the architecture's own config.json keys, and a function
from that configuration to a `ModelSpec` (the parts of every layer, the order
in which layers run, the tensor names).  The reference has no registry (one
package per architecture); this one is this package's own design.
"""
from __future__ import annotations

import dataclasses
from typing import Callable

from .base import ConfigError, ModelConfig, read_config_json


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_spec: Callable  # (config) -> parts.ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}' (registered: {', '.join(known_architectures()) or 'none'})")
    return _ARCHITECTURES[name]


def config_from_dict(raw: dict, where: str = "config.json") -> ModelConfig:
    archs = raw.get("architectures")
    if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
        raise ConfigError(f"{where}: key 'architectures' must be a list that names the model class")
    return lookup_architecture(archs[0]).config_class.from_dict(raw, where)


def load_config(folder: str) -> ModelConfig:
    import os
    return config_from_dict(read_config_json(folder), os.path.join(folder, "config.json"))
