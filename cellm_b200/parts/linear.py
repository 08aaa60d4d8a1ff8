"""A weight matrix [out, in] applied as x . W^T (no bias: the reference's
linears have none, crates/cellm-model/src/lfm.rs:924-981)."""
from __future__ import annotations

import torch

from .. import ops


class Linear:
    def __init__(self, weight: torch.Tensor, act_dtype: torch.dtype):
        self.weight = weight.contiguous()
        self.act_dtype = act_dtype
        self.out_features, self.in_features = self.weight.shape

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        out_dtype = out_dtype or self.act_dtype
        if self.weight.dtype == x.dtype:
            return ops.gemm(x, self.weight, out_dtype)
        # A matrix kept in 32-bit under bfloat16 activations runs the 32-bit product.
        y = ops.gemm(x.to(self.weight.dtype), self.weight, torch.float32)
        return y if out_dtype == torch.float32 else y.to(out_dtype)


def stack_rows(*mats: torch.Tensor) -> torch.Tensor:
    """Several [n_i, K] matrices as one [sum n_i, K], so one product serves all."""
    dt = mats[0].dtype
    if any(m.dtype != dt for m in mats):
        mats = [m.to(torch.float32) for m in mats]
    return torch.cat(list(mats), dim=0).contiguous()
