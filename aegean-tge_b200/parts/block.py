"""Arrangements of a mixer and a feed-forward around the residual stream."""
from __future__ import annotations

import torch

from .base import BLOCKS, Block, LayerCache, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x)).

    The stream ``x`` is float32 and is never itself normalised: each norm's
    output feeds the part and the part's output is added back
    (src/models/qwen2.cpp:2055, :2099-2105, :2118).
    """

    passes_deferred_rows = True

    def forward(self, x, ctx: StepContext, cache: LayerCache, h=None, next_norm=None, next_takes_deferred=False):
        if h is None:
            h = self.mixer_norm.forward(x)
        # a part is only asked to leave the norm's factor to its successor if both sides say they can
        defer = {"defer": True} if self.mixer.can_defer_norm and self.feed_forward.takes_deferred_rows else {}
        h = self.mixer.forward_add(h, x, ctx, cache, next_norm=self.ffn_norm, **defer)
        if h is None:
            h = self.ffn_norm.forward(x)
        defer = {"defer": True} if self.feed_forward.can_defer_norm and next_takes_deferred else {}
        return self.feed_forward.forward_add(h, x, ctx, next_norm=next_norm, **defer)
