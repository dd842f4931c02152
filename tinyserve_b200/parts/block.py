"""Pre-norm residual block: ``x += mixer(norm(x)); x += feed_forward(norm(x))``
(upstream src/tinyserve/model.py:154-179). The two sums are not made here: each sub-layer's
output is left pending on the stream and the next norm adds it in 32-bit.
"""

from __future__ import annotations

from typing import Any

from .base import Block, ResidualStream, StepContext, register_block


class PreNormBlock(Block):
    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Any, writes_cache: bool,
                position: Any) -> None:
        # Scratch of this layer goes to the other half of the arena than the previous
        # layer's, whose pending output the first norm below still has to read.
        ctx.arena.next_frame()
        hn = self.mixer_norm.forward(stream, ctx)
        mixed = self.mixer.forward(hn, ctx, cache, writes_cache, position)
        stream.delta = mixed
        hn = self.feed_forward_norm.forward(stream, ctx)
        stream.delta = self.feed_forward.forward(hn, ctx)


register_block("prenorm", PreNormBlock)
