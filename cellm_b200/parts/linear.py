"""A weight matrix [out, in] applied as x . W^T (no bias: the reference's
linears have none, crates/cellm-model/src/lfm.rs:924-981)."""
from __future__ import annotations

import torch

from .. import ops
from ..ops.gemm_bf16 import FoldAfter, FoldBefore, can_fold
from .base import Prescaled, ResidualSink


def fold_after(x, weight: torch.Tensor, epilogue: int = 0):
    """(input tensor, FoldAfter or None) for a product whose input may be a Prescaled:
    the norm's scale moves into the product where its tiles allow, else the normed
    rows are formed first."""
    if not isinstance(x, Prescaled):
        return x, None
    u = x.u
    if weight.dtype == torch.bfloat16 and u.dtype == torch.bfloat16 and ops.tensor_core_ok(u, weight) \
            and can_fold(u.shape[0], weight.shape[0], u.shape[1], u.device, epilogue):
        return u, FoldAfter(x.parts, x.dim, x.eps)
    return x.materialize(), None


class Linear:
    def __init__(self, weight: torch.Tensor, act_dtype: torch.dtype):
        self.weight = weight.contiguous()
        self.act_dtype = act_dtype
        self.out_features, self.in_features = self.weight.shape

    def __call__(self, x, out_dtype: torch.dtype | None = None, sink: ResidualSink | None = None):
        """x . W^T. `x` may be a Prescaled (a norm's unformed output). With `sink` the
        output may be added to the residual stream here, for the norm that follows;
        None is returned then."""
        out_dtype = out_dtype or self.act_dtype
        x, after = fold_after(x, self.weight)
        if sink is not None and self.weight.dtype == x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 \
                and ops.tensor_core_ok(x, self.weight) and sink.residual.pending is None \
                and tuple(sink.residual.x.shape) == (x.shape[0], self.out_features) \
                and can_fold(x.shape[0], self.out_features, self.in_features, x.device):
            u, parts = ops.gemm(x, self.weight, out_dtype, w_is_static=True,
                                before=FoldBefore(sink.residual.x, sink.norm.weight), after=after)
            sink.delivered(u, parts)
            return None
        if self.weight.dtype == x.dtype:
            return ops.gemm(x, self.weight, out_dtype, w_is_static=True, after=after)
        # A matrix kept in 32-bit under bfloat16 activations runs the 32-bit product.
        y = ops.gemm(x.to(self.weight.dtype), self.weight, torch.float32)
        return y if out_dtype == torch.float32 else y.to(out_dtype)


def stack_rows(*mats: torch.Tensor) -> torch.Tensor:
    """Several [n_i, K] matrices as one [sum n_i, K], so one product serves all."""
    dt = mats[0].dtype
    if any(m.dtype != dt for m in mats):
        mats = [m.to(torch.float32) for m in mats]
    return torch.cat(list(mats), dim=0).contiguous()
