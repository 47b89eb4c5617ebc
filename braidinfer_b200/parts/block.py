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
        x = self._norm(self.mixer_norm, h, ctx, self.mixer)
        h = self.mixer.forward(x, h, ctx, cache, state)
        if self.feed_forward is not None:
            x = self._norm(self.feed_forward_norm, h, ctx, self.feed_forward)
            h = self.feed_forward.forward(x, h, ctx)
        if ctx.row_scales:
            raise RuntimeError("a part left a row scale unapplied (see StepContext.row_scales)")
        return h

    @staticmethod
    def _norm(norm, h, ctx, reader):
        if not norm.accepts_deferred:
            return norm.forward(ctx.resolve(h), ctx)
        # a norm that knows deferred sums may also leave its scale to a reader that takes row scales
        return norm.forward(h, ctx, reader_takes_row_scale=bool(reader.takes_row_scale()))
