"""Arrangements of a layer's parts around the residual stream.

'pre_norm' (``src/model/qwen3/model.cpp:779-923``):  h += mixer(norm1(h));  h += feed_forward(norm2(h)).
The residual sum is 32-bit; each add is fused into the norm that follows it, so a block leaves its
last sub-layer's output pending on the stream - unless the sub-layer added it itself: a part that says so
(``adds_to_residual``) is handed the residual and the norm that comes next, and may hand back that norm's
input already prepared (``ops.NormedRows``); a part that says ``takes_deferred_norm`` is given it instead of
the norm's result.  With both, a decode step runs no norm kernel and no add between the products.
"""
from __future__ import annotations

from .. import ops
from .base import Block, ResidualStream, register_part


def _fusable(norm):
    f = norm.fusable() if norm is not None and hasattr(norm, "fusable") else None
    return None if f is None else (f[0], f[1], norm)


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    capturable = True       # see parts.base.Part.capturable
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _normed(norm, part, stream: ResidualStream, ctx):
        prepared, stream.prepared = stream.prepared, None
        if (prepared is not None and prepared.owner is norm and stream.pending is None
                and getattr(part, "takes_deferred_norm", False)):
            return prepared
        x = norm.add_norm(stream.hidden, stream.pending, ctx, upcoming=part.first_weights())
        stream.pending = None
        return x

    @staticmethod
    def _run(part, args, stream: ResidualStream, next_norm) -> None:
        if getattr(part, "adds_to_residual", False):
            out = part.forward(*args, residual=stream.hidden, next_norm=_fusable(next_norm))
        else:
            out = part.forward(*args)
        if isinstance(out, ops.NormedRows):
            stream.prepared, stream.pending = out, None
        else:
            stream.pending = out          # a tensor still to be added, or None: the part added it itself

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        after = stream.next_norm
        x = self._normed(self.mixer_norm, self.mixer, stream, ctx)
        ctx.upcoming_weights = self.feed_forward.first_weights()      # for the mixer's last small kernel
        self._run(self.mixer, (x, ctx, cache), stream, self.feed_forward_norm)
        ctx.upcoming_weights = None
        x = self._normed(self.feed_forward_norm, self.feed_forward, stream, ctx)
        self._run(self.feed_forward, (x, ctx), stream, after)
