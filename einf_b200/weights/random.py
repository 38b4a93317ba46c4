"""Random weights: a model folder from a configuration and a seed.

The reference has no such mode (its tests rely on ``nn.Linear`` default
initialisation under ``torch.manual_seed``, ``tests/test_torch_qwen.py:72-75``).
Matrices and biases are drawn N(0, ``init_std``), norm weights
1 + N(0, ``init_scale_std``), one tensor after another in sorted name order
from one seeded CPU generator, and stored in bfloat16, so every reader of the
folder sees the same values.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch
from safetensors.torch import save_file

from ..config.base import ModelConfig
from ..config.specs import TensorSpec


def random_tensors(
    expected: Mapping[str, TensorSpec],
    seed: int,
    std: float = 0.02,
    scale_std: float = 0.05,
    dtype: torch.dtype = torch.bfloat16,
    device: str | torch.device = "cpu",
) -> dict[str, torch.Tensor]:
    """One random tensor for each expected name.

    On the CPU the values depend on the seed only; on a CUDA device they are
    drawn there (fast for large models) and differ from the CPU stream.
    """
    device = torch.device(device)
    generator = torch.Generator(device=device)
    generator.manual_seed(seed)
    tensors = {}
    for name in sorted(expected):
        spec = expected[name]
        if spec.role == "table":
            raise ValueError(f"no random rule for integer table {name}")
        values = torch.randn(spec.shape, generator=generator, dtype=torch.float32, device=device)
        if spec.role == "scale":
            values = 1.0 + scale_std * values
        else:
            values = std * values
        tensors[name] = values.to(dtype)
    return tensors


def write_random_model(
    folder: str | Path,
    config: ModelConfig,
    seed: int,
    dtype: torch.dtype = torch.bfloat16,
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``folder``."""
    from ..parts.model import expected_tensors  # parts declare their tensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    expected, _ = expected_tensors(config.model_spec())
    tensors = random_tensors(expected, seed, config.init_std, config.init_scale_std, dtype)
    (folder / "config.json").write_text(json.dumps(config.to_dict(), indent=1), encoding="utf-8")
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
