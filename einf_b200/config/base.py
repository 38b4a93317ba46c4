"""Base class of typed model configurations.

A configuration is a frozen dataclass whose fields are the keys of the
architecture's own ``config.json``.  ``from_dict`` refuses a missing required
key by name, as the reference does (``src/einf/executors/torch/qwen.py:93-117``
indexes the dict and raises ``KeyError``), and ``model_spec`` turns the values
into the part-by-part description the rest of the engine reads.
"""
from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Any, ClassVar

from .specs import ModelSpec


class ConfigError(ValueError):
    """A config.json that is missing a key or holds a value the engine refuses."""


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    #: the string found in ``config.json["architectures"][0]``
    architecture: ClassVar[str] = ""
    #: keys that would change what the model computes but that this class does not compute:
    #: key -> the values under which it changes nothing.  Any other value is refused by name
    #: (keys that are neither fields nor listed here are informational and ignored).
    refused_keys: ClassVar[dict[str, tuple]] = {}

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "ModelConfig":
        values: dict[str, Any] = {}
        missing: list[str] = []
        for f in dataclasses.fields(cls):
            if f.name in data:
                values[f.name] = data[f.name]
            elif f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING:
                missing.append(f.name)
        if missing:
            raise ConfigError(
                f"config.json of {cls.architecture} lacks required key(s): {', '.join(missing)}"
            )
        for key, harmless in cls.refused_keys.items():
            if key in data and data[key] not in harmless:
                raise ConfigError(
                    f"config.json of {cls.architecture} sets {key} = {data[key]!r}, which this engine does "
                    f"not compute; it would run the model without it and give wrong logits"
                )
        config = cls(**values)
        config.validate()
        return config

    @classmethod
    def from_json(cls, path: str | Path) -> "ModelConfig":
        return cls.from_dict(json.loads(Path(path).read_text(encoding="utf-8")))

    def to_dict(self) -> dict[str, Any]:
        data = {"architectures": [self.architecture]}
        data.update(dataclasses.asdict(self))
        return data

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError

    # Values the engine needs from every architecture.
    @property
    def eos_token_ids(self) -> tuple[int, ...]:
        return ()

    @property
    def init_std(self) -> float:
        """Standard deviation of random matrices and biases in the random-weights mode."""
        return 0.02

    @property
    def init_scale_std(self) -> float:
        """Standard deviation around 1 of random norm weights in the random-weights mode."""
        return 0.05
