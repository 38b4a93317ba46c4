"""Sampling: parameters and the device sampler."""
from .params import GREEDY, SamplingParams
from .sampler import Sampler

__all__ = ["GREEDY", "Sampler", "SamplingParams"]
