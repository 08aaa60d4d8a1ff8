"""SwiGLU feed-forward (crates/cellm-model/src/lfm.rs:631-662):
W2 (silu(W1 m) * (W3 m)), no biases. W1 and W3 are stacked so that one
product yields gate and up side by side."""
from __future__ import annotations

import torch

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
        self.ff, self.H, self.dtype = ff, H, dtype
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
        self._record = None

    def record(self):
        """The part as an op record of the native executor (None: its weights do not fit the activations'
        element type, and forward() below runs it kernel by kernel)."""
        from ..runtime import records as R
        if self._record is None and self.gate_up.weight.dtype == self.dtype == self.down.weight.dtype:
            self._record = R.Record(R.SWIGLU, R.SwiGLUParams(R.linear(self.gate_up.weight), R.linear(self.down.weight),
                                                             self.ff, int(self.fused)), part=self)
        return self._record

    def emit(self, emitter) -> None:
        rec = self.record()
        if rec is None:
            return super().emit(emitter)
        emitter.records.append(rec)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        from .. import ops
        from ..runtime.program import part_program
        rec = self.record()
        if rec is not None:
            return part_program(self.dtype, x.device, self.H).run_part(rec, x, ctx)
        # matrices kept in another element type than the activations: product, gate, product
        gu = self.gate_up(x, out_dtype=torch.float32)
        return self.down(ops.swiglu(gu, self.dtype))


register_feed_forward("swiglu", SwiGLU)
