"""Pre-norm arrangement of a layer (crates/cellm-model/src/lfm.rs:333-347,
:610-629, :665-667): x += mixer(norm(x)); x += feed_forward(norm(x))."""
from __future__ import annotations

from typing import Optional

from .base import Block, CacheBinding, Norm, Residual, StepContext
from .registry import register_block


class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding, next_norm: Optional[Norm] = None) -> None:
        mixer, ff = self.mixer, self.feed_forward
        ff_lazy = getattr(ff, "takes_prescaled", False)
        x = self.mixer_norm.forward(residual, prescaled_ok=getattr(mixer, "takes_prescaled", False))
        # the mixer's last product may add to the stream itself if the feed-forward can read what it leaves
        ctx.sink = self.feed_forward_norm.sink(residual, ctx.T) if ff_lazy and getattr(mixer, "feeds_sink", False) else None
        out = mixer.forward(x, ctx, cache)
        ctx.sink = None
        residual.add(out)
        x = self.feed_forward_norm.forward(residual, prescaled_ok=ff_lazy)
        # likewise the feed-forward's, for the norm after this block (its reader is asked by whoever runs it)
        ctx.sink = next_norm.sink(residual, ctx.T) if next_norm is not None and getattr(ff, "feeds_sink", False) else None
        out = ff.forward(x, ctx)
        ctx.sink = None
        residual.add(out)

    def first_norm(self) -> Optional[Norm]:
        return self.mixer_norm

    def first_takes_prescaled(self) -> bool:
        return getattr(self.mixer, "takes_prescaled", False)


register_block("pre_norm", PreNormBlock)
