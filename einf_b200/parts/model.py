"""A decoder model put together from a :class:`ModelSpec`.

The model owns its parts and the order they run in; it does not own the cache.
``cache_plan`` says which run of which layer needs what, and the engine gives
``forward`` one :class:`CacheView` per schedule entry.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from ..config.specs import ModelSpec, PartSpec, TensorSpec
from .base import (
    CacheView, PagedKVNeed, Runtime, StateNeed, StepContext, build_part, part_class, walk_part_specs,
)
from .block import build_block


def _part_specs(model_spec: ModelSpec):
    """Every (category, PartSpec) of the model, with the parts that parts of any category nest."""
    yield from walk_part_specs("embedding", model_spec.embedding)
    for layer in model_spec.layers:
        block_class = part_class("block", layer.block)
        for role, category in block_class.part_categories().items():
            yield from walk_part_specs(category, layer.parts[role])
    yield from walk_part_specs("norm", model_spec.final_norm)
    yield from walk_part_specs("head", model_spec.head)


def expected_tensors(model_spec: ModelSpec) -> tuple[dict[str, TensorSpec], dict[str, TensorSpec]]:
    """Checkpoint tensors the model needs, and those it tolerates (a stored copy of a tied matrix)."""
    expected: dict[str, TensorSpec] = {}
    for category, spec in _part_specs(model_spec):
        for name, tensor_spec in part_class(category, spec.kind).tensor_specs(spec).items():
            expected[spec.prefix + name] = tensor_spec
    optional: dict[str, TensorSpec] = {}
    head = model_spec.head
    if head.get("tied_to"):
        optional[head.prefix + "weight"] = TensorSpec((head["vocab_size"], head["hidden_size"]))
    return expected, optional


def kernel_libraries(model_spec: ModelSpec, runtime: Runtime) -> tuple[str, ...]:
    names: list[str] = []
    for category, spec in _part_specs(model_spec):
        names.extend(part_class(category, spec.kind).kernel_libraries(spec, runtime))
    return tuple(dict.fromkeys(names))


@dataclass(frozen=True)
class EntryCache:
    """Cache of one schedule entry: ``owner`` is the entry whose storage it uses."""

    need: PagedKVNeed | StateNeed | None
    owner: int
    group: int = -1   # page group of a paged need


@dataclass(frozen=True)
class CachePlan:
    entries: tuple[EntryCache, ...]
    #: window of each page group (None: all keys are kept)
    group_windows: tuple[Optional[int], ...]

    @property
    def has_state(self) -> bool:
        return any(isinstance(e.need, StateNeed) for e in self.entries)


class DecoderModel:
    def __init__(self, model_spec: ModelSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.spec = model_spec
        self.runtime = runtime
        self.embedding = build_part("embedding", model_spec.embedding, tensors, runtime)
        self.blocks = [build_block(layer, tensors, runtime) for layer in model_spec.layers]
        self.final_norm = build_part("norm", model_spec.final_norm, tensors, runtime)
        head_spec = model_spec.head
        head_class = part_class("head", head_spec.kind)
        tied = None
        if head_spec.get("tied_to"):
            if head_spec["tied_to"] != model_spec.embedding.prefix + "weight":
                raise ValueError(f"head is tied to {head_spec['tied_to']!r}, which is not the embedding table")
            tied = self.embedding.table
            self.head = head_class(head_spec, {}, runtime, tied=tied)
        else:
            self.head = build_part("head", head_spec, tensors, runtime)
        self.schedule = model_spec.schedule
        self.cache_plan = self._plan_cache()

    def _plan_cache(self) -> CachePlan:
        windows: list[Optional[int]] = []
        entries: list[EntryCache] = []
        for index, entry in enumerate(self.schedule):
            need = self.blocks[entry.layer].mixer.cache_need()
            owner = index if entry.cache_from is None else entry.cache_from
            if owner != index:
                owner_need = entries[owner].need
                if type(owner_need) is not type(need) or (
                    isinstance(need, PagedKVNeed)
                    and (need.num_kv_heads, need.head_size) != (owner_need.num_kv_heads, owner_need.head_size)
                ):
                    raise ValueError(
                        f"schedule entry {index} cannot read the cache of entry {owner}: {need} vs {owner_need}"
                    )
            group = -1
            if isinstance(need, PagedKVNeed):
                if owner != index:
                    group = entries[owner].group
                else:
                    if need.window not in windows:
                        windows.append(need.window)
                    group = windows.index(need.window)
            entries.append(EntryCache(need, owner, group))
        if not windows:
            windows.append(None)  # the manager always has one page group
        return CachePlan(tuple(entries), tuple(windows))

    def forward(self, ctx: StepContext, caches: list[CacheView]) -> torch.Tensor:
        """Run the step's tokens through every schedule entry; float logits ``[S, vocab]``
        at ``ctx.logit_rows``."""
        residual = self.embedding.forward(ctx)
        pending = None
        for index, entry in enumerate(self.schedule):
            pending = self.blocks[entry.layer].forward(residual, pending, ctx, caches[index])
        if getattr(self.final_norm, "takes_status", False):
            x = self.final_norm.forward(pending, residual, rows=ctx.logit_rows, status=ctx.status)
        else:
            x = self.final_norm.forward(pending, residual, rows=ctx.logit_rows)
        return self.head.forward(x, ctx.status)
