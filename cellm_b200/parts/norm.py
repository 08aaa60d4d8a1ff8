"""RMSNorm (crates/cellm-kernels/src/cpu_kernels.rs:17-34): x / sqrt(mean(x^2) + eps) * w,
fused with the addition of whatever waits to be added to the residual stream."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, Residual, TensorSpec
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

    def emit(self, emitter) -> None:
        from ..ops._lib import tag
        from ..runtime import records as R
        emitter.native(R.RMS_NORM, R.RmsNormParams(self.weight.data_ptr(), tag(self.weight), self.eps), part=self)

    def forward(self, residual: Residual, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        delta, residual.pending = residual.pending, None
        y = ops.add_rmsnorm(residual.x, delta, self.weight, self.eps, self.dtype, rows)
        if rows is not None and delta is not None:
            residual.pending = delta      # the stream itself was not updated
        return y


register_norm("rms_norm", RMSNorm)
