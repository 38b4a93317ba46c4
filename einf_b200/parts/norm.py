"""RMSNorm fused with the residual add.

``residual += pending; out = weight * residual * rsqrt(mean(residual^2) + eps)``,
all in 32-bit, rounded once into the activation type: the reference's
``fused_add_rmsnorm`` (``src/einf/executors/torch/fused_ops.py:41-68``; weight
initialised to ones, eps inside the root, ``qwen.py:125-132``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import Norm, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    @classmethod
    def tensor_specs(cls, spec):
        return {"weight": TensorSpec((spec["size"],), "scale")}

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = runtime.vector(tensors["weight"])

    #: ``forward`` takes the step's status word (``status=``), where a kernel with a bounded wait reports
    takes_status = True

    def forward(self, pending, residual, rows: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None):
        count = rows.shape[0] if rows is not None else residual.shape[0]
        out = torch.empty((count, self.size), dtype=self.runtime.dtype, device=residual.device)
        ops.add_rmsnorm(pending, residual, self.weight, self.eps, out, rows, status)
        return out
