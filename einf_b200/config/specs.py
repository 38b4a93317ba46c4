"""Declarative description of a model: parts, layers, and the order they run in.

A configuration class turns the keys of its ``config.json`` into a
:class:`ModelSpec`.  Everything below it (weights, parts, cache, step
function) reads only the spec: no part knows which architecture it is in.

The reference hard-wires one decoder class (``src/einf/executors/torch/qwen.py:492-593``);
here the same information is data so that layers may differ from one another.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


def _freeze(params: Mapping[str, Any]) -> Mapping[str, Any]:
    return MappingProxyType(dict(params))


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: which implementation (``kind``) and its constants.

    ``prefix`` is the checkpoint name prefix of the part's tensors, e.g.
    ``model.layers.3.self_attn.``; a part only knows its local tensor names.
    """

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""

    def __post_init__(self) -> None:
        object.__setattr__(self, "params", _freeze(self.params))

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)

    def with_prefix(self, prefix: str) -> "PartSpec":
        return PartSpec(self.kind, self.params, prefix)


@dataclass(frozen=True)
class LayerSpec:
    """A block: the arrangement (``block``) and the parts it arranges."""

    block: str
    parts: Mapping[str, PartSpec]

    def __post_init__(self) -> None:
        object.__setattr__(self, "parts", _freeze(self.parts))


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer inside a step.

    ``layer`` indexes :attr:`ModelSpec.layers`; naming it twice runs the same
    weights twice.  Each entry owns a cache of its own unless ``cache_from``
    names an earlier entry: then it reads that entry's cache and writes none.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec

    def __post_init__(self) -> None:
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(
                    f"schedule entry {index} names layer {entry.layer}, "
                    f"but the model has {len(self.layers)} layers"
                )
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < index:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry "
                        f"{entry.cache_from}, which does not run before it"
                    )
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(
                        f"schedule entry {index} reads the cache of entry "
                        f"{entry.cache_from}, which owns no cache itself"
                    )


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects from the checkpoint.

    ``role`` drives the random-weights mode only: ``matrix`` and ``bias`` are
    drawn N(0, std), ``scale`` (norm weights) 1 + N(0, std).
    """

    shape: tuple[int, ...]
    role: str = "matrix"
