"""Gated short convolution mixer (crates/cellm-model/src/lfm.rs:350-417):
in_proj to B | C | x, B*x, a causal depthwise convolution over the last `taps`
values of B*x, times C, out_proj. Its per-request state is the last taps-1
values of B*x, in a slot of fixed size."""
from __future__ import annotations

import torch

from ..config.errors import ConfigError
from .base import CacheBinding, FixedState, Mixer, StepContext, TensorSpec
from .linear import Linear
from .registry import register_mixer


class ShortConvMixer(Mixer):
    graph_safe = True

    """params: hidden_size, taps, bias. weights: in_proj [3H, H], conv [H, 1, taps],
    out_proj [H, H], conv_bias [H] if bias."""

    @classmethod
    def weight_specs(cls, params):
        H, taps = params["hidden_size"], params["taps"]
        specs = {"in_proj": TensorSpec((3 * H, H), "linear"), "conv": TensorSpec((H, 1, taps), "conv_tap"),
                 "out_proj": TensorSpec((H, H), "linear")}
        if params.get("bias"):
            specs["conv_bias"] = TensorSpec((H,), "bias")
        return specs

    @classmethod
    def cache_need(cls, params):
        return FixedState((max(int(params["taps"]) - 1, 0), int(params["hidden_size"])), torch.float32)

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.H, self.taps, self.dtype = int(params["hidden_size"]), int(params["taps"]), dtype
        if not 1 <= self.taps <= 16:
            raise ConfigError(f"short_conv: {self.taps} taps; the kernel takes 1 to 16")
        self.in_proj = Linear(weights["in_proj"], dtype)
        self.out_proj = Linear(weights["out_proj"], dtype)
        self.conv_w = weights["conv"].reshape(self.H, self.taps).contiguous()
        self.conv_b = None
        if params.get("bias"):
            self.conv_b = weights["conv_bias"].to(self.conv_w.dtype).contiguous()
        # Decode steps (one token per request) run in_proj and the convolution as one kernel, which reads
        # in_proj in tiles that keep a channel's B, C and x rows together: a second copy of that matrix.
        from ..ops import gemm_bf16 as tc
        self.in_proj_tiled = None
        w = self.in_proj.weight
        if (dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and self.conv_w.dtype == torch.bfloat16
                and self.taps <= tc.CONV_MAX_TAPS and self.H % 8 == 0):
            self.in_proj_tiled = tc.tile_in_proj_for_conv(w)
        self._record = None

    def record(self):
        """The part as an op record of the native executor (None: its matrices are kept in another element type
        than the activations)."""
        from ..ops._lib import tag
        from ..runtime import records as R
        if self._record is None and self.in_proj.weight.dtype == self.dtype == self.out_proj.weight.dtype:
            p = R.ShortConvParams(R.linear(self.in_proj.weight), R.linear(self.out_proj.weight))
            if self.in_proj_tiled is not None:
                p.in_proj_tiled, p.tiled_rows = self.in_proj_tiled.data_ptr(), self.in_proj_tiled.shape[0]
            p.taps, p.bias = self.conv_w.data_ptr(), R.ptr(self.conv_b)
            p.taps_dtype, p.n_taps = tag(self.conv_w), self.taps
            self._record = R.Record(R.SHORT_CONV, p, part=self)
        return self._record

    def emit(self, emitter) -> None:
        rec = self.record()
        if rec is None:
            return super().emit(emitter)
        emitter.records.append(rec)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        from .. import ops
        from ..runtime.program import part_program
        rec = self.record()
        if rec is not None:
            return part_program(self.dtype, x.device, self.H).run_part(rec, x, ctx, cache)
        bcx = self.in_proj(x)
        y = ops.short_conv(bcx, self.conv_w, self.conv_b, cache.state, ctx.slot_ids, ctx.seq_of_token,
                           ctx.cu_seqlens, ctx.err, ctx.max_q_len)
        return self.out_proj(y)


register_mixer("short_conv", ShortConvMixer)
