"""Pre-norm residual block: ``x += mixer(norm(x)); x += feed_forward(norm(x))``
(upstream src/tinyserve/model.py:154-179). The two sums are not made here: each sub-layer's
output is left pending on the stream and the next norm adds it in 32-bit.
"""

from __future__ import annotations

from typing import Any, Mapping

from .base import Block, Part, ResidualStream, StepContext, register_block


class PreNormBlock(Block):
    # the order is the order of the layer's tensors in ``tensor_specs``
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, parts: Mapping[str, Part]) -> None:
        super().__init__(parts)
        self.mixer, self.feed_forward = parts["mixer"], parts["feed_forward"]
        self.mixer_norm, self.feed_forward_norm = parts["mixer_norm"], parts["feed_forward_norm"]

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, Any], writes_cache: bool,
                position: Any) -> None:
        # Scratch of this layer goes to the other half of the arena than the previous
        # layer's, whose pending output the first norm below still has to read.
        ctx.arena.next_frame()
        mixer, ff = self.mixer, self.feed_forward
        cache = caches.get("mixer")
        ctx.upcoming_weights = ff.streamed_weights()
        hn = self.mixer_norm.lazy(stream, ctx) if mixer.takes_lazy_input else self.mixer_norm.forward(stream, ctx)
        if mixer.adds_to_stream:
            mixed = mixer.forward(hn, ctx, cache, writes_cache, position, stream=stream)
        else:
            mixed = mixer.forward(hn, ctx, cache, writes_cache, position)
        self._leave(stream, mixed)
        hn = self.feed_forward_norm.lazy(stream, ctx) if ff.takes_lazy_input else self.feed_forward_norm.forward(stream, ctx)
        self._leave(stream, ff.forward(hn, ctx, stream=stream) if ff.adds_to_stream else ff.forward(hn, ctx))

    @staticmethod
    def _leave(stream: ResidualStream, out: Any) -> None:
        """A sub-layer's output stays pending on the stream, unless the part has added it itself."""
        if out is not None:
            stream.delta = out
            stream.sumsq = None


register_block("prenorm", PreNormBlock)
