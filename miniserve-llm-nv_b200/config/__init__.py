"""Typed configuration and the architecture registry."""

from .engine_config import EngineConfig
from .model_config import BafavikConfig, KivuraxConfig, Qwen3Config, VesidraConfig, ZozezenConfig
from .registry import (Architecture, UnsupportedModelError, load_model_config, read_config_json,
                       register_architecture, registered_architectures, resolve_architecture)

__all__ = ["Architecture", "BafavikConfig", "EngineConfig", "KivuraxConfig", "Qwen3Config", "VesidraConfig", "ZozezenConfig", "UnsupportedModelError", "load_model_config",
           "read_config_json", "register_architecture", "registered_architectures", "resolve_architecture"]
