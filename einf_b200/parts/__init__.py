"""Parts of a model and the model assembled from them."""
from . import attention, block, embedding, mlp, norm, position  # noqa: F401  (registers the kinds)
from .base import (
    CacheView,
    FeedForward,
    Mixer,
    Norm,
    PagedKVNeed,
    Part,
    Runtime,
    StateNeed,
    StepContext,
    build_nested,
    build_part,
    known_parts,
    part_class,
    register_part,
)
from .block import Block, PreNormBlock, build_block
from .model import CachePlan, DecoderModel, EntryCache, expected_tensors, kernel_libraries

__all__ = [
    "Block",
    "CachePlan",
    "CacheView",
    "DecoderModel",
    "EntryCache",
    "FeedForward",
    "Mixer",
    "Norm",
    "PagedKVNeed",
    "Part",
    "PreNormBlock",
    "Runtime",
    "StateNeed",
    "StepContext",
    "build_block",
    "build_nested",
    "build_part",
    "expected_tensors",
    "kernel_libraries",
    "known_parts",
    "part_class",
    "register_part",
]
