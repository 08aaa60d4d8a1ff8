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

    BLOCK = 64      # rows per gate / up block in the layout of the fused kernel

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        w1, w3 = weights["w1"], weights["w3"]
        ff, H = w1.shape
        # bfloat16 with a width that is a multiple of 64: gate and up rows are
        # interleaved block by block, so that the product's epilogue has a gate and
        # its up side by side and applies silu(g) * u before anything is stored.
        self.fused = (dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and w3.dtype == torch.bfloat16
                      and ff % self.BLOCK == 0 and H % 8 == 0)
        if self.fused:
            b = self.BLOCK
            blocked = torch.stack([w1.reshape(ff // b, b, H), w3.reshape(ff // b, b, H)], dim=1).reshape(2 * ff, H)
            self.gate_up = Linear(blocked.contiguous(), dtype)
        else:
            self.gate_up = Linear(stack_rows(w1, w3), dtype)
        self.down = Linear(weights["w2"], dtype)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        if self.fused and x.dtype == torch.bfloat16 and ops.tensor_core_ok(x, self.gate_up.weight):
            return self.down(ops.gemm_swiglu_bf16(x, self.gate_up.weight, w_is_static=True))
        if self.fused:
            raise ValueError("swiglu: activations do not fit the fused kernel (bfloat16, 16-byte aligned rows)")
        return self.down(ops.swiglu(self.gate_up(x)))


register_feed_forward("swiglu", SwiGLU)
