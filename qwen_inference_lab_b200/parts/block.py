"""Arrangement of a layer's parts: norm -> mixer -> + -> norm -> feed-forward -> +.

The pre-norm order of the reference's ``DecoderBlock.forward`` (qil/model.py:48-71).
The block owns no sizes: it is given a norm, a mixer, a second norm and a
feed-forward, each already built, so different layers of one model may hold
different kinds of each.
"""
from __future__ import annotations

from .base import Part


class PreNormBlock(Part):
    def __init__(self, mixer_norm, mixer, ff_norm, feed_forward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.ff_norm, self.feed_forward = ff_norm, feed_forward
        self.graph_safe = True

    def children(self):
        return [self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward]

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, ctx, x, cache):
        """x [N, hidden] is the residual stream; returned updated (possibly in place)."""
        if getattr(self.mixer, "takes_norm", False):
            x = self.mixer.forward(ctx, x, cache, residual=x, norm=self.mixer_norm)
        else:
            x = self.mixer.forward(ctx, self.mixer_norm.forward(ctx, x), cache, residual=x)
        if getattr(self.feed_forward, "takes_norm", False):
            return self.feed_forward.forward(ctx, x, residual=x, norm=self.ff_norm)
        return self.feed_forward.forward(ctx, self.ff_norm.forward(ctx, x), residual=x)
