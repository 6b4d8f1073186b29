"""Arrangements of a layer's parts.

``pre_norm``: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(model/llama.go:1087-1097, 1311-1314, 1425).  Its parameters are the four
nested specs ``mixer_norm``, ``mixer``, ``feed_forward_norm`` and
``feed_forward``.  The additions are not done here: each update is left
pending on the residual stream and the next norm (of this layer, of the next
one, or the final one) adds it in float32 while it normalises -- unless the
part, offered the stream (`emit_update`), has added its update in its last
product's epilogue already and returns None.
"""
from __future__ import annotations

from ..cache import CacheHandle
from .base import Block, ResidualStream, StepContext, register_part


def _hidden(stream: ResidualStream):
    """The hidden state as a value: the residual with its pending update added."""
    if stream.pending is None:
        return stream.residual.clone()
    return stream.residual + stream.pending.float()


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    sub_parts = (("mixer_norm", "norm"), ("mixer", "mixer"),
                 ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: CacheHandle) -> None:
        ctx.trace("hidden_in", lambda: _hidden(stream))
        x = self.mixer_norm.forward(stream, ctx)
        ctx.trace("normed", x)
        ctx.update_into = stream
        try:
            stream.pending = self.mixer.forward(x, ctx, cache)
            if stream.pending is not None:
                ctx.trace("o", stream.pending)
            x = self.feed_forward_norm.forward(stream, ctx)
            ctx.trace("mlp_input", x)
            stream.pending = self.feed_forward.forward(x, ctx)
            if stream.pending is not None:
                ctx.trace("down", stream.pending)
        finally:
            ctx.update_into = None
        ctx.trace("hidden_post_ffn", lambda: _hidden(stream))
