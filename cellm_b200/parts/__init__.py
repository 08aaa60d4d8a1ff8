"""Importing this package registers the built-in parts."""
from .base import (Block, CacheBinding, FeedForward, FixedState, Mixer, Norm, PagedKV, Part, Position,
                   Residual, StepContext, TensorSpec)
from .registry import (part_class, register_block, register_feed_forward, register_mixer, register_norm,
                       register_position, registered)
from . import attention, block, norm, rope, short_conv, swiglu  # noqa: F401
