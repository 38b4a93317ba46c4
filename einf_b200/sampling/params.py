"""Sampling parameters: the C++ ``SamplingParams`` of the control plane.

Names, defaults and checks follow the reference
(``crates/einf-control/src/sample.rs:22-108``): ``temperature`` 0 means greedy
and then takes no ``top_k``/``top_p``/``min_p``; ``top_k`` None or positive;
``top_p`` in (0, 1]; ``min_p`` in [0, 1]; ``seed``; ``stop_token_ids``.
"""
from ..cache.control import SamplingParams

GREEDY = SamplingParams()

__all__ = ["GREEDY", "SamplingParams"]
