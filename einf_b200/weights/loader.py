"""Weights from safetensors by tensor name.

The reference reads ``model.safetensors`` or the shards named by
``model.safetensors.index.json`` into one dict and hands it to
``load_state_dict(strict=True)`` (``src/einf/executors/torch/qwen.py:698-727``).
Here the expected names and shapes come from the parts of the model, and every
disagreement is gathered into one :class:`WeightsError`.

Storage policy: floating tensors are kept in bfloat16, except that a tensor the
file stores in 32-bit stays 32-bit; integer tables become int32.  Parts ask
for the precision they compute in when they take a tensor.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch
from safetensors import safe_open

from ..config.specs import TensorSpec

_FLOAT32_LIKE = (torch.float32, torch.float64)
_INTEGERS = (torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64, torch.bool)


class WeightsError(RuntimeError):
    """The tensors of a folder do not match what the model expects."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_kind=()):
        self.missing = tuple(missing)
        self.unexpected = tuple(unexpected)
        self.wrong_shape = tuple(wrong_shape)
        self.wrong_kind = tuple(wrong_kind)
        lines = ["weights do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, found, expected in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(found)}, expected {list(expected)}")
        for name, found in self.wrong_kind:
            lines.append(f"  wrong kind: {name} is {found}, expected a floating tensor")
        super().__init__("\n".join(lines))


def kept_dtype(stored: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in, given the dtype the file stores."""
    if stored in _FLOAT32_LIKE:
        return torch.float32
    if stored in _INTEGERS:
        return torch.int32
    return torch.bfloat16


def shard_files(folder: str | Path) -> list[Path]:
    """The safetensors files of a model folder (``qwen.py:703-715``)."""
    folder = Path(folder)
    if folder.is_file():
        return [folder]
    single = folder / "model.safetensors"
    if single.is_file():
        return [single]
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text(encoding="utf-8"))["weight_map"]
        return [folder / name for name in sorted(set(weight_map.values()))]
    raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json in {folder}")


def load_tensors(
    folder: str | Path,
    expected: Mapping[str, TensorSpec],
    device: str | torch.device = "cpu",
    optional: Mapping[str, TensorSpec] | None = None,
) -> dict[str, torch.Tensor]:
    """Read exactly the ``expected`` tensors; raise one error naming every fault.

    ``optional`` tensors are taken and checked if present (a tied output matrix
    that a folder stores anyway) and ignored otherwise.
    """
    optional = optional or {}
    found: dict[str, torch.Tensor] = {}
    unexpected: list[str] = []
    wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]] = []
    wrong_kind: list[tuple[str, str]] = []
    for path in shard_files(folder):
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for name in handle.keys():
                spec = expected.get(name) or optional.get(name)
                if spec is None:
                    unexpected.append(name)
                    continue
                shape = tuple(handle.get_slice(name).get_shape())
                if shape != tuple(spec.shape):
                    wrong_shape.append((name, shape, tuple(spec.shape)))
                    continue
                tensor = handle.get_tensor(name)
                if spec.role != "table" and not tensor.is_floating_point():
                    wrong_kind.append((name, str(tensor.dtype)))
                    continue
                found[name] = tensor.to(kept_dtype(tensor.dtype)).to(device)
    bad = {name for name, _, _ in wrong_shape} | {name for name, _ in wrong_kind}
    missing = [name for name in expected if name not in found and name not in bad]
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightsError(sorted(missing), sorted(unexpected), wrong_shape, wrong_kind)
    return found
