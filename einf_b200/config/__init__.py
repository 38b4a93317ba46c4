"""Typed configurations and the architecture registry."""
from .base import ConfigError, ModelConfig
from .engine import EngineConfig
from .qwen2 import Qwen2Config
from .registry import (
    config_class_for,
    config_from_dict,
    known_architectures,
    load_config,
    register_architecture,
)
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec

register_architecture(Qwen2Config)

__all__ = [
    "ConfigError",
    "EngineConfig",
    "LayerSpec",
    "ModelConfig",
    "ModelSpec",
    "PartSpec",
    "Qwen2Config",
    "ScheduleEntry",
    "TensorSpec",
    "config_class_for",
    "config_from_dict",
    "known_architectures",
    "load_config",
    "register_architecture",
]
