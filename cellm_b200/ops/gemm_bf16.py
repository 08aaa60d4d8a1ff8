from __future__ import annotations

import torch

from .gemm import gemm_plain


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """bfloat16 product with 32-bit accumulation."""
    return gemm_plain(a, w, out_dtype)
