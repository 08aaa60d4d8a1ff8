"""Importing this package registers the built-in parts."""
from .base import (Block, CacheBinding, Embedding, FeedForward, FixedState, Head, Mixer, Norm, PagedKV, Part, Position,
                   Residual, StepContext, TensorSpec)
from .registry import (part_class, register_block, register_embedding, register_feed_forward, register_head,
                       register_mixer, register_norm, register_position, registered)
from . import attention, block, embedding, norm, rope, short_conv, swiglu  # noqa: F401
