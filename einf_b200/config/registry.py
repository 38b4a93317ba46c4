"""One registry from an architecture's name to its configuration class.

The reference imports its one model class directly (``scripts/run_qwen.py:14,88``)
and has no registry.  Here ``config.json["architectures"][0]`` picks the
configuration class; the class's ``model_spec`` then names the parts, so
adding an architecture is one ``register_architecture`` call.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any

from .base import ConfigError, ModelConfig

_ARCHITECTURES: dict[str, type[ModelConfig]] = {}


def register_architecture(config_class: type[ModelConfig]) -> type[ModelConfig]:
    name = config_class.architecture
    if not name:
        raise ValueError(f"{config_class.__name__} declares no architecture name")
    known = _ARCHITECTURES.get(name)
    if known is not None and known is not config_class:
        raise ValueError(f"architecture {name!r} is already registered to {known.__name__}")
    _ARCHITECTURES[name] = config_class
    return config_class


def known_architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def config_class_for(name: str) -> type[ModelConfig]:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def config_from_dict(data: dict[str, Any]) -> ModelConfig:
    architectures = data.get("architectures")
    if not isinstance(architectures, (list, tuple)) or not architectures:
        raise ConfigError("config.json has no 'architectures' list naming the model class")
    return config_class_for(str(architectures[0])).from_dict(data)


def load_config(path: str | Path) -> ModelConfig:
    """Read ``config.json`` from a model folder (or the file itself)."""
    path = Path(path)
    if path.is_dir():
        path = path / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json at {path}")
    return config_from_dict(json.loads(path.read_text(encoding="utf-8")))
