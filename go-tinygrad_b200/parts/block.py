"""Arrangements of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(model/llama.go:1087-1097, 1311-1314, 1425).  The additions are not done here:
each update is left pending on the residual stream and the next norm (of this
layer, of the next one, or the final one) adds it in float32 while it
normalises -- unless the part, offered the stream (`emit_update`), has added
its update in its last product's epilogue already and returns None.
"""
from __future__ import annotations

from ..cache import CacheHandle
from .base import Block, ResidualStream, StepContext, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        x = self.mixer_norm.forward(stream, ctx)
        ctx.update_into = stream
        try:
            stream.pending = self.mixer.forward(x, ctx, cache)
            x = self.ff_norm.forward(stream, ctx)
            stream.pending = self.ff.forward(x, ctx)
        finally:
            ctx.update_into = None
