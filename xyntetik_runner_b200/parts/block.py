"""Pre-norm block: x -> norm -> mixer -> +x -> norm -> feed-forward -> +x
(src/model.c:6206-6208, 6350-6352, 6366-6368, 6421-6423).  The two additions happen in float32
inside the last product of the mixer and of the feed-forward."""
from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm, register_block


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ff_norm: Norm, feed_forward: FeedForward):
        self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward = mixer_norm, mixer, ff_norm, feed_forward

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    def tensors(self):
        out = {}
        for p in self.parts():
            out.update(p.tensors())
        return out

    def bind(self, tensors, rt):
        for p in self.parts():
            p.bind(tensors, rt)

    def weight_bytes(self):
        return sum(p.weight_bytes() for p in self.parts())

    def forward(self, ctx, x, lay):
        # A norm finishes whatever sum the part before it left pending on x (see StepContext.set_pending),
        # so x is complete whenever a mixer or a feed-forward runs.
        h = ctx.buf("block_normed", (x.shape[0], x.shape[1]), ctx.act_dtype)
        self.mixer_norm.forward(ctx, x, h)
        self.mixer.forward(ctx, h, x, lay)
        self.ff_norm.forward(ctx, x, h)
        self.feed_forward.forward(ctx, h, x)


register_block("prenorm", PreNormBlock)
