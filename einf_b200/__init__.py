"""einf_b200: a small, whole LLM inference engine for one NVIDIA B200.

From a model folder (``config.json`` + safetensors) to generated tokens on one
GPU: typed configuration and architecture registry, weights by tensor name,
layers assembled from parts, a paged cache with per-request block tables, one
step function over mixed batches, a scheduler, sampling, and hand-written
sm_100a kernels.
"""

__version__ = "0.1.0"
