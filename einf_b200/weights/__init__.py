"""Weights: read by tensor name from safetensors, or drawn at random."""
from .loader import WeightsError, kept_dtype, load_tensors, shard_files
from .random import random_tensors, write_random_model

__all__ = [
    "WeightsError",
    "kept_dtype",
    "load_tensors",
    "random_tensors",
    "shard_files",
    "write_random_model",
]
