"""The two ends of the model: token embedding and the output matrix.

``embedding``: ``h0[t] = table[token[t]]``, no scaling
(``src/einf/executors/torch/qwen.py:744``), written straight into the 32-bit
residual stream.  ``linear_head``: ``logits = x @ W^T`` without bias, in 32-bit
output; with ``tied_to`` it uses that tensor (the embedding table) instead of
one of its own (``qwen.py:690-696``).  The reference computes logits for every
token (``qwen.py:772-773``); here only the wanted rows reach the head.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import Part, register_part


@register_part("embedding", "embedding")
class TokenEmbedding(Part):
    @classmethod
    def tensor_specs(cls, spec):
        return {"weight": TensorSpec((spec["vocab_size"], spec["hidden_size"]))}

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.table = runtime.matrix(tensors["weight"])
        self.hidden_size = int(spec["hidden_size"])

    def forward(self, ctx) -> torch.Tensor:
        residual = torch.empty((ctx.num_tokens, self.hidden_size), dtype=torch.float32, device=self.table.device)
        ops.embed(ctx.token_ids, self.table, residual, ctx.status)
        return residual


@register_part("head", "linear_head")
class LinearHead(Part):
    @classmethod
    def tensor_specs(cls, spec):
        if spec.get("tied_to"):
            return {}
        return {"weight": TensorSpec((spec["vocab_size"], spec["hidden_size"]))}

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("gemm_simt",) + (("gemm_tcgen05",) if runtime.dtype == torch.bfloat16 else ())

    def __init__(self, spec, tensors, runtime, tied=None):
        super().__init__(spec, tensors, runtime)
        self.vocab_size = int(spec["vocab_size"])
        self.weight = tied if tied is not None else runtime.matrix(tensors["weight"])

    def forward(self, x: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        return ops.project(x, self.weight, status, out_dtype=torch.float32, allow_partial=False)
