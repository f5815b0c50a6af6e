"""Typed configurations read from a model folder's config.json.

A configuration class names the config.json keys of its architecture, their
defaults and the checks on them; no size lives anywhere else.  `KeyReader`
collects every problem of a config.json into one error.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any


class ConfigError(ValueError):
    """A config.json that this package cannot use; the message lists every fault."""


_MISSING = object()


class KeyReader:
    """Reads keys of a config.json dict and remembers what went wrong."""

    def __init__(self, raw: dict, where: str = "config.json"):
        self.raw = raw
        self.where = where
        self.problems: list[str] = []

    def get(self, key: str, kind, default: Any = _MISSING):
        v = self.raw.get(key, None)
        if v is None:
            if default is _MISSING:
                self.problems.append(f"missing key '{key}'")
                return kind() if kind in (int, float, bool, str) else None
            return default
        if kind is float and isinstance(v, (int, float)) and not isinstance(v, bool):
            return float(v)
        if kind is int and isinstance(v, bool):
            self.problems.append(f"key '{key}' must be an integer, got {v!r}")
            return 0
        if kind is int and isinstance(v, float) and v == int(v):
            return int(v)
        if not isinstance(v, kind):
            self.problems.append(f"key '{key}' must be {kind.__name__}, got {v!r}")
            return kind()
        return v

    def require(self, cond: bool, message: str) -> None:
        if not cond:
            self.problems.append(message)

    def finish(self) -> None:
        if self.problems:
            raise ConfigError(f"{self.where}: " + "; ".join(self.problems))


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration."""
    architecture: str

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        """The config.json that reads back to this configuration."""
        raise NotImplementedError

    def stop_token_ids(self) -> tuple[int, ...]:
        return ()


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.exists(path):
        raise ConfigError(f"{path}: no such file")
    with open(path) as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw
