"""Typed configurations and the architecture registry."""
from .base import ConfigError, ModelConfig, read_config_json
from .qwen3 import Qwen3Config
from .registry import (Architecture, config_from_dict, known_architectures, load_config, lookup_architecture,
                       register_architecture)
from . import qwen3_model  # noqa: F401,E402  (registers Qwen3ForCausalLM)

__all__ = ["Architecture", "ConfigError", "ModelConfig", "Qwen3Config", "config_from_dict", "known_architectures",
           "load_config", "lookup_architecture", "read_config_json", "register_architecture"]
