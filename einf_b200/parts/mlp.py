"""Gated feed-forward: ``down(act(gate(x)) * up(x))``.

Gate and up share one matrix product on the concatenated weight, gate rows
first (``src/einf/executors/torch/qwen.py:163-172,206-208``); the activation is
SiLU (``fused_ops.py:71-77``), the only one Qwen2 uses (``qwen.py:138-139``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import FeedForward, register_part


@register_part("feed_forward", "gated_mlp")
class GatedMLP(FeedForward):
    @classmethod
    def tensor_specs(cls, spec):
        hidden, inter = spec["hidden_size"], spec["intermediate_size"]
        return {
            "gate_proj.weight": TensorSpec((inter, hidden)),
            "up_proj.weight": TensorSpec((inter, hidden)),
            "down_proj.weight": TensorSpec((hidden, inter)),
        }

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise", "gemm_simt") + (("gemm_tcgen05",) if runtime.dtype == torch.bfloat16 else ())

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp has a SiLU kernel only, not {spec['activation']!r}")
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if gate.dtype != up.dtype:
            gate, up = gate.to(torch.float32), up.to(torch.float32)
        self.gate_up_weight = runtime.matrix(torch.cat([gate, up], dim=0))
        self.down_weight = runtime.matrix(tensors["down_proj.weight"])

    def forward(self, x, ctx):
        tokens = x.shape[0]
        dtype, device = self.runtime.dtype, x.device
        gate_up = ops.project(x, self.gate_up_weight, ctx.status)   # [T, 2I], or split-K partial sums
        hidden = torch.empty((tokens, self.intermediate_size), dtype=dtype, device=device)
        ops.silu_mul(gate_up, hidden)
        return ops.project(hidden, self.down_weight, ctx.status)
