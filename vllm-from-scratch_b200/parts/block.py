"""Arrangement of a layer's parts around the residual stream.

``pre_norm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))``, written with
the not-yet-added output carried beside the residual so that every addition is
fused into the next norm (minivllm/models/qwen3.py:216-233).

For steps of a few tokens, where the mixer and the feed-forward say that they split norms
(:meth:`~.base.Mixer.splits_norms`), neither norm runs as a kernel of its own: the product
ahead of a norm adds into the residual and hands on :class:`~.base.HalfNormedRows`, the
product behind it applies the root; the second product of the feed-forward does so under
the next block's first norm."""

from __future__ import annotations

import torch

from .base import BLOCKS, Block, CacheView, HalfNormedRows, Norm, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    norm_roles = ("mixer", "feed_forward")
    graph_safe = True

    def _splits_norms(self, tokens: int) -> bool:
        return (self.norms["feed_forward"].split() is not None and self.mixer.splits_norms(tokens)
                and self.feed_forward.splits_norms(tokens))

    def first_norm(self) -> Norm:
        return self.norms["mixer"]

    def takes_half_normed(self, tokens: int) -> bool:
        return self.norms["mixer"].split() is not None and self._splits_norms(tokens)

    def folds_into(self, norm: Norm, tokens: int) -> bool:
        return norm.split() is not None and self._splits_norms(tokens)

    def forward(self, x: torch.Tensor | HalfNormedRows | None, residual: torch.Tensor, ctx: StepContext,
                cache: CacheView, next_norm: Norm | None = None) -> torch.Tensor | HalfNormedRows:
        normed = x if isinstance(x, HalfNormedRows) else self.norms["mixer"].forward(x, residual)
        if not self._splits_norms(residual.shape[0]):
            mixed = self.mixer.forward(normed, ctx, cache)
            normed = self.norms["feed_forward"].forward(mixed, residual)
            return self.feed_forward.forward(normed, ctx)
        half = self.mixer.forward(normed, ctx, cache, fold=(residual, self.norms["feed_forward"]))
        return self.feed_forward.forward(half, ctx, fold=None if next_norm is None else (residual, next_norm))
