"""Arrangements of a layer's parts.

"prenorm_residual": h = h + mixer(norm(h)); h = h + feed_forward(norm(h)), the
order of the reference's attention-plus-dense layer
(crates/braidinfer-runtime/src/megakernel/megakernel_compile.rs:115-236).  The
residual stream h is float32; mixers and feed-forwards add into it.
"""
from __future__ import annotations

from .base import BLOCKS, Block


@BLOCKS.register("prenorm_residual")
class PreNormResidualBlock(Block):
    def forward(self, h, ctx, cache, state):
        # h may still wait for a deferred sum (see StepContext.deferred); a norm that
        # accepts that adds it up in its own kernel, any other part gets h completed first
        if not self.mixer_norm.accepts_deferred:
            ctx.resolve(h)
        x = self.mixer_norm.forward(h, ctx)
        h = self.mixer.forward(x, h, ctx, cache, state)
        if self.feed_forward is not None:
            if not self.feed_forward_norm.accepts_deferred:
                ctx.resolve(h)
            x = self.feed_forward_norm.forward(h, ctx)
            h = self.feed_forward.forward(x, h, ctx)
        return h
