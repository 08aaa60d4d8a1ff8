"""Pre-norm arrangement of a layer (crates/cellm-model/src/lfm.rs:333-347,
:610-629, :665-667): x += mixer(norm(x)); x += feed_forward(norm(x))."""
from __future__ import annotations

from .base import Block, CacheBinding, Residual, StepContext
from .registry import register_block


class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def emit(self, emitter) -> None:
        """The layer as records: each of the four parts emits its own, in the order they run."""
        for part in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward):
            part.emit(emitter)

    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding) -> None:
        residual.add(self.mixer.forward(self.mixer_norm.forward(residual), ctx, cache))
        residual.add(self.feed_forward.forward(self.feed_forward_norm.forward(residual), ctx))


register_block("pre_norm", PreNormBlock)
