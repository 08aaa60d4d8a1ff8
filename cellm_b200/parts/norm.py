"""RMSNorm (crates/cellm-kernels/src/cpu_kernels.rs:17-34): x / sqrt(mean(x^2) + eps) * w,
fused with the addition of whatever waits to be added to the residual stream."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, Prescaled, Residual, ResidualSink, TensorSpec
from .registry import register_norm


class RMSNorm(Norm):
    graph_safe = True

    """params: dim, eps. weights: weight [dim]."""

    @classmethod
    def weight_specs(cls, params):
        return {"weight": TensorSpec((params["dim"],), "norm")}

    def __init__(self, params: dict, weights: dict, dtype: torch.dtype):
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])
        self.weight = weights["weight"].contiguous()
        self.dtype = dtype

    FOLD_MAX_TOKENS = 64          # the products' tiles that can take a norm's half hold at most this many tokens

    def forward(self, residual: Residual, rows: Optional[torch.Tensor] = None, prescaled_ok: bool = False):
        folded, residual.folded = residual.folded, None
        if folded is not None and folded[0] is self and residual.pending is None and rows is None:
            # the product before has added its output and left u = stream * weight and the sums of squares
            plain = lambda: ops.add_rmsnorm(residual.x, None, self.weight, self.eps, self.dtype)
            return Prescaled(folded[1], folded[2], self.dim, self.eps, plain) if prescaled_ok else plain()
        delta, residual.pending = residual.pending, None
        y = ops.add_rmsnorm(residual.x, delta, self.weight, self.eps, self.dtype, rows)
        if rows is not None and delta is not None:
            residual.pending = delta      # the stream itself was not updated
        return y

    def sink(self, residual: Residual, T: int) -> Optional[ResidualSink]:
        if self.dtype != torch.bfloat16 or T > self.FOLD_MAX_TOKENS or residual.x.shape[1] != self.dim:
            return None
        return ResidualSink(residual, self)


register_norm("rms_norm", RMSNorm)
