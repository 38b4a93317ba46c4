"""Grouped-query attention over the paged cache.

One matrix product for Q, K and V on the concatenated weight
(``src/einf/executors/torch/packed_qkv.py:70-107,135-153``); bias, position
encoding and the cache write in one kernel; every token of the step attends to
the keys of its own request through the block table, so a prompt portion sees
itself through the cache (``qwen.py:405-411``); query head ``h`` uses key/value
head ``h // (heads / kv_heads)``; scores are scaled by ``scale`` and masked
lower-right causal (``model_runner.py:145``), optionally to the last ``window``
keys; then the output projection (``qwen.py:360,489``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import CacheView, Mixer, PagedKVNeed, StepContext, build_nested, register_part


@register_part("mixer", "attention")
class PagedAttention(Mixer):
    @classmethod
    def tensor_specs(cls, spec):
        hidden, heads, kv_heads, size = (
            spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_size"],
        )
        specs = {
            "q_proj.weight": TensorSpec((heads * size, hidden)),
            "k_proj.weight": TensorSpec((kv_heads * size, hidden)),
            "v_proj.weight": TensorSpec((kv_heads * size, hidden)),
            "o_proj.weight": TensorSpec((hidden, heads * size)),
        }
        if spec.get("qkv_bias", False):
            specs["q_proj.bias"] = TensorSpec((heads * size,), "bias")
            specs["k_proj.bias"] = TensorSpec((kv_heads * size,), "bias")
            specs["v_proj.bias"] = TensorSpec((kv_heads * size,), "bias")
        if spec.get("out_bias", False):
            specs["o_proj.bias"] = TensorSpec((hidden,), "bias")
        return specs

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        if ops.has_fast_attention(runtime.dtype, int(spec["head_size"])):
            # the page size is the engine's choice: ask for both prefill kernels of this head size
            libraries = ops.attention_libraries(int(spec["head_size"]), 16)
            return ("pointwise", "gemm_simt", "gemm_tcgen05") + libraries
        return ("pointwise", "attention_generic", "gemm_simt") + cls._product_libraries(runtime)

    @staticmethod
    def _product_libraries(runtime):
        return ("gemm_tcgen05",) if runtime.dtype == torch.bfloat16 else ()

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.head_size = int(spec["head_size"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} key/value heads")
        if self.head_size % 16 or self.head_size > ops.MAX_HEAD_SIZE:
            raise ops.UnsupportedSize(
                f"head size {self.head_size}: the attention kernels take multiples of 16 up to {ops.MAX_HEAD_SIZE}"
            )
        if self.window is not None and self.window <= 0:
            raise ValueError(f"window must be positive, got {self.window}")
        matrices = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        if len({m.dtype for m in matrices}) > 1:
            matrices = [m.to(torch.float32) for m in matrices]
        self.qkv_weight = runtime.matrix(torch.cat(matrices, dim=0))
        self.qkv_bias = None
        if spec.get("qkv_bias", False):
            self.qkv_bias = runtime.vector(
                torch.cat([tensors["q_proj.bias"].float(), tensors["k_proj.bias"].float(), tensors["v_proj.bias"].float()])
            )
        self.out_weight = runtime.matrix(tensors["o_proj.weight"])
        self.out_bias = runtime.vector(tensors["o_proj.bias"]) if spec.get("out_bias", False) else None
        self.position = build_nested("position", spec["position"], tensors, runtime)
        self.fast = ops.has_fast_attention(runtime.dtype, self.head_size)

    def cache_need(self):
        return PagedKVNeed(self.num_kv_heads, self.head_size, self.window)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens = x.shape[0]
        dtype, device = self.runtime.dtype, x.device
        qkv = ops.project(x, self.qkv_weight, ctx.status)   # [T, width], or split-K partial sums
        q = torch.empty((tokens, self.num_heads, self.head_size), dtype=dtype, device=device)
        self.position.encode_and_store(
            qkv, self.qkv_bias, ctx, cache, q, self.num_heads, self.num_kv_heads, self.head_size
        )
        mixed = torch.empty_like(q)
        self.attend(q, ctx, cache, mixed)
        if self.out_bias is None:
            return ops.project(mixed.view(tokens, -1), self.out_weight, ctx.status)
        out = torch.empty((tokens, self.hidden_size), dtype=dtype, device=device)
        ops.linear(mixed.view(tokens, -1), self.out_weight, self.out_bias, out)
        return out

    def launch_key(self, ctx: StepContext, page_size: int) -> tuple:
        """The decode attention cuts a token's keys by the number of single tokens and the bucket
        of the longest context: kernel, cluster size and clusters per token."""
        singles = int(ctx.single_tokens.shape[0])
        if not self.fast or not singles:
            return ()
        context = min(ctx.max_context_len, self.window) if self.window else ctx.max_context_len
        return ops.decode_plan(singles, self.num_heads, self.num_kv_heads, self.head_size, page_size, context)

    def launch_group(self):
        return ("attention", self.num_heads, self.num_kv_heads, self.head_size, self.window, self.fast)

    def attend(self, q, ctx: StepContext, cache: CacheView, out) -> None:
        """bfloat16 with a head size up to 128: the tensor-core kernels, cluster decode for the
        requests that bring one token, tiled prefill for the others, side by side in a mixed batch.  Everything else (the 32-bit path,
        larger heads): the generic kernel."""
        table = ctx.block_tables[cache.group]
        if self.fast:
            singles = ctx.single_tokens.shape[0]
            if singles:
                ops.paged_decode_attention_auto(
                    q, cache.k, cache.v, table, ctx.seq_of_token, ctx.positions, out, self.scale,
                    self.window, ctx.status, None if ctx.decode_only else ctx.single_tokens,
                    max_context=ctx.max_context_len,
                )
            if ctx.q_tiles.shape[0]:
                ops.paged_prefill_attention(
                    q, cache.k, cache.v, table, ctx.q_tiles, out, self.scale, self.window, ctx.status,
                    cached_before=ctx.max_portion_start,
                )
            return
        ops.paged_attention_generic(
            q, cache.k, cache.v, ctx.block_tables[cache.group], ctx.seq_of_token, ctx.positions,
            out, self.scale, self.window, ctx.status,
        )
