"""Position encodings.  The attention mixer hands its raw QKV rows to the
position part, which adds the bias, encodes Q and K, and stores K and V in the
pages: one kernel does all three, so Q, K and V are read once.

``rope``: rotate-half rotary encoding over the first ``rotary_dim`` dims of each
head, ``inv_freq[i] = theta^(-2i/rotary_dim)``, angle ``position * inv_freq[i]``
in 32-bit (``src/einf/executors/torch/model_runner.py:42-78``).  The table of
inverse frequencies is made on the host by the reference's own expression, so
that angles agree with a host computation bit for bit.

``none``: no encoding; bias and the cache write only.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, register_part


class PositionEncoding(Part):
    def encode_and_store(self, qkv, bias, ctx, cache, q_out, num_heads, num_kv_heads, head_size):
        raise NotImplementedError


def _store(inv_freq, qkv, bias, ctx, cache, q_out, num_heads, num_kv_heads, head_size):
    writes = cache is not None and cache.writes and cache.k is not None
    ops.rope_kv_write(
        qkv,
        bias,
        ctx.positions,
        inv_freq,
        ctx.slots[cache.group] if writes else None,
        q_out,
        cache.k if writes else None,
        cache.v if writes else None,
        num_heads,
        num_kv_heads,
        head_size,
        ctx.status,
    )


@register_part("position", "rope")
class RotaryPosition(PositionEncoding):
    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        if self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even")
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2).float() / self.rotary_dim))
        self.inv_freq = inv_freq.to(runtime.device)

    def encode_and_store(self, qkv, bias, ctx, cache, q_out, num_heads, num_kv_heads, head_size):
        if self.rotary_dim > head_size:
            raise ValueError(f"rotary_dim {self.rotary_dim} exceeds head size {head_size}")
        _store(self.inv_freq, qkv, bias, ctx, cache, q_out, num_heads, num_kv_heads, head_size)


@register_part("position", "none")
class NoPosition(PositionEncoding):
    @classmethod
    def kernel_libraries(cls, spec, runtime):
        return ("pointwise",)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.inv_freq = torch.empty(0, dtype=torch.float32, device=runtime.device)

    def encode_and_store(self, qkv, bias, ctx, cache, q_out, num_heads, num_kv_heads, head_size):
        _store(self.inv_freq, qkv, bias, ctx, cache, q_out, num_heads, num_kv_heads, head_size)
