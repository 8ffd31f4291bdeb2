"""Typed configuration and the architecture registry."""

from .engine_config import EngineConfig
from .model_config import Qwen3Config
from .registry import (Architecture, UnsupportedModelError, load_model_config, read_config_json,
                       register_architecture, registered_architectures, resolve_architecture)

__all__ = ["Architecture", "EngineConfig", "Qwen3Config", "UnsupportedModelError", "load_model_config",
           "read_config_json", "register_architecture", "registered_architectures", "resolve_architecture"]
