"""Arrangements of parts in one layer.

``prenorm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))``.  The
residual stream ``h`` is a 32-bit tensor; a sublayer's output stays *pending*
until the next norm adds it, so each add is fused with the norm that follows
(``src/einf/executors/torch/qwen.py:526-563``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import CacheView, Part, StepContext, build_part, part_class, register_part


class Block(Part):
    mixer: Part

    @classmethod
    def part_categories(cls) -> dict[str, str]:
        """Role name in :class:`LayerSpec.parts` -> part category."""
        raise NotImplementedError

    def forward(
        self, residual: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext, cache: CacheView
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """Consume ``pending`` into the residual stream and return ``(residual, pending)``: the
        stream as it stands now (``residual`` updated in place, or another tensor) and the
        output that the next norm is to add."""
        raise NotImplementedError


@register_part("block", "prenorm")
class PreNormBlock(Block):
    @classmethod
    def part_categories(cls):
        return {
            "mixer_norm": "norm",
            "mixer": "mixer",
            "feed_forward_norm": "norm",
            "feed_forward": "feed_forward",
        }

    def __init__(self, layer_spec, tensors, runtime):
        self.runtime = runtime
        self.spec = layer_spec
        for role, category in self.part_categories().items():
            setattr(self, role, build_part(category, layer_spec.parts[role], tensors, runtime))
        # A sublayer that starts with a matrix product may absorb the weight of the norm before
        # it; at few tokens it then runs straight from the residual stream, with no norm kernel.
        for norm, part in ((self.mixer_norm, self.mixer), (self.feed_forward_norm, self.feed_forward)):
            weight = norm.foldable_weight() if hasattr(norm, "foldable_weight") else None
            fold = getattr(part, "fold_input_scale", None)
            if weight is not None and fold is not None and fold(weight):
                norm.drop_weight()

    @staticmethod
    def _from_residual(part, num_tokens, pending) -> bool:
        takes = getattr(part, "takes_residual", None)
        return takes is not None and takes(num_tokens, pending)

    def forward(self, residual, pending, ctx, cache):
        if self._from_residual(self.mixer, ctx.num_tokens, pending):
            mixed, residual = self.mixer.forward_from_residual(pending, residual, self.mixer_norm.eps, ctx, cache)
        else:
            x = self.mixer_norm.forward(pending, residual)
            mixed = self.mixer.forward(x, ctx, cache)
        if self._from_residual(self.feed_forward, ctx.num_tokens, mixed):
            out, residual = self.feed_forward.forward_from_residual(mixed, residual, self.feed_forward_norm.eps, ctx)
        else:
            x = self.feed_forward_norm.forward(mixed, residual)
            out = self.feed_forward.forward(x, ctx)
        return residual, out


def build_block(layer_spec, tensors, runtime) -> Block:
    return part_class("block", layer_spec.block)(layer_spec, tensors, runtime)
