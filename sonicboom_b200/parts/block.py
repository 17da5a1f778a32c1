"""Arrangement of parts in a block.  "pre_norm": h = norm(x); x1 = mix(h) + x; f = norm(x1);
x2 = ffn(f) + x1 (core/src/model/emit.cpp:436-459 with no post norms, gate or output scale,
as the reference's traits set for this architecture: core/src/model/recipe.cpp:65-70)."""
from __future__ import annotations

from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, make, register_block)


@register_block("pre_norm")
class PreNormBlock(Block):
    def __init__(self, spec, dtype, device):
        self.dtype = dtype
        self.mixer_norm = make(NORMS, "norm", spec.mixer_norm, dtype, device)
        self.mixer = make(MIXERS, "mixer", spec.mixer, dtype, device)
        self.feed_forward_norm = make(NORMS, "norm", spec.feed_forward_norm, dtype, device)
        self.feed_forward = make(FEED_FORWARDS, "feed-forward", spec.feed_forward, dtype, device)
        self.parts = [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def tensor_requests(self):
        return [r for p in self.parts for r in p.tensor_requests()]

    def bind(self, get):
        for p in self.parts:
            p.bind(get)

    def kv_need(self):
        return self.mixer.kv_need()

    def state_need(self):
        return self.mixer.state_need()

    def input_norm(self):
        return self.mixer_norm

    def first_weights(self, rows):
        return self.mixer.first_weights(rows)

    def forward(self, x, ctx):
        h = ctx.take_normed(self.mixer_norm, x)
        if h is None:
            h = self.mixer_norm.forward(x, self.dtype)
        ctx.next_norm = self.feed_forward_norm
        x = self.mixer.forward(h, ctx, residual=x)
        f = ctx.take_normed(self.feed_forward_norm, x)
        if f is None:
            f = self.feed_forward_norm.forward(x, self.dtype)
        # the block's result is the feed-forward's, so what follows the block follows its product
        ctx.next_norm, ctx.next_weights = ctx.after_block_norm, ctx.after_block_weights
        return self.feed_forward.forward(f, ctx, residual=x)
