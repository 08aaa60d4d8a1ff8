"""SwiGLU feed-forward (crates/cellm-model/src/lfm.rs:631-662):
W2 (silu(W1 m) * (W3 m)), no biases. W1 and W3 are stacked so that one
product yields gate and up side by side."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, StepContext, TensorSpec
from .linear import Linear, stack_rows
from .registry import register_feed_forward


class SwiGLU(FeedForward):
    graph_safe = True

    """params: hidden_size, ff_dim. weights: w1, w3 [ff, H]; w2 [H, ff]."""

    @classmethod
    def weight_specs(cls, params):
        H, ff = params["hidden_size"], params["ff_dim"]
        return {"w1": TensorSpec((ff, H), "linear"), "w3": TensorSpec((ff, H), "linear"),
                "w2": TensorSpec((H, ff), "linear")}

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.gate_up = Linear(stack_rows(weights["w1"], weights["w3"]), dtype)
        self.down = Linear(weights["w2"], dtype)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return self.down(ops.swiglu(self.gate_up(x)))


register_feed_forward("swiglu", SwiGLU)
