"""Arrangements of a layer's parts around the residual stream.

'pre_norm' (``src/model/qwen3/model.cpp:779-923``):  h += mixer(norm1(h));  h += feed_forward(norm2(h)).
The residual sum is 32-bit; each add is fused into the norm that follows it, so a block leaves its
last sub-layer's output pending on the stream.
"""
from __future__ import annotations

from .base import Block, ResidualStream, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self.mixer_norm.add_norm(stream.hidden, stream.pending, ctx, upcoming=self.mixer.first_weights())
        ctx.upcoming_weights = self.feed_forward.first_weights()      # for the mixer's last small kernel
        stream.pending = self.mixer.forward(x, ctx, cache)
        ctx.upcoming_weights = None
        x = self.feed_forward_norm.add_norm(stream.hidden, stream.pending, ctx, upcoming=self.feed_forward.first_weights())
        stream.pending = self.feed_forward.forward(x, ctx)
