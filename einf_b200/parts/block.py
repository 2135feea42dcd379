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
    ) -> torch.Tensor:
        """Consume ``pending`` into ``residual`` and return the new pending output."""
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

    @staticmethod
    def _normalise(norm, pending, residual, ctx):
        # a norm that declares ``takes_status`` gets the step's status word as well
        if getattr(norm, "takes_status", False):
            return norm.forward(pending, residual, status=ctx.status)
        return norm.forward(pending, residual)

    def forward(self, residual, pending, ctx, cache):
        x = self._normalise(self.mixer_norm, pending, residual, ctx)
        mixed = self.mixer.forward(x, ctx, cache)
        x = self._normalise(self.feed_forward_norm, mixed, residual, ctx)
        return self.feed_forward.forward(x, ctx)


@register_part("block", "prenorm_mixer")
class PreNormMixerBlock(PreNormBlock):
    """``h += mixer(norm1(h))`` and nothing else: a layer without a feed-forward."""

    @classmethod
    def part_categories(cls):
        return {"mixer_norm": "norm", "mixer": "mixer"}

    def forward(self, residual, pending, ctx, cache):
        x = self._normalise(self.mixer_norm, pending, residual, ctx)
        return self.mixer.forward(x, ctx, cache)


@register_part("block", "parallel")
class ParallelBlock(PreNormBlock):
    """``h += mixer(n) + feed_forward(n)`` with one norm ``n = norm(h)`` that both sublayers read.
    A feed-forward that takes an addend sums both in its last kernel, in 32-bit; otherwise the
    pending value is the stack of both as float32 terms, which the next norm adds up."""

    @classmethod
    def part_categories(cls):
        return {"mixer_norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

    def forward(self, residual, pending, ctx, cache):
        x = self._normalise(self.mixer_norm, pending, residual, ctx)
        mixed = self.mixer.forward(x, ctx, cache)
        if getattr(self.feed_forward, "takes_addend", False):
            return self.feed_forward.forward(x, ctx, add=mixed)   # its last kernel adds the two up
        terms = [mixed if mixed.dim() == 3 else mixed[None], self.feed_forward.forward(x, ctx)[None]]
        return torch.cat([term.to(torch.float32) for term in terms], dim=0)


def build_block(layer_spec, tensors, runtime) -> Block:
    return part_class("block", layer_spec.block)(layer_spec, tensors, runtime)
