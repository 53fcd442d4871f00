"""Arrangement of a layer's parts around the residual stream.

``pre_norm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))``, written with
the not-yet-added output carried beside the residual so that every addition is
fused into the next norm (minivllm/models/qwen3.py:216-233)."""

from __future__ import annotations

import torch

from .base import BLOCKS, Block, CacheView, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    norm_roles = ("mixer", "feed_forward")
    graph_safe = True

    def forward(self, x: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                cache: CacheView) -> torch.Tensor:
        normed = self.norms["mixer"].forward(x, residual)
        mixed = self.mixer.forward(normed, ctx, cache)
        normed = self.norms["feed_forward"].forward(mixed, residual)
        return self.feed_forward.forward(normed, ctx)
