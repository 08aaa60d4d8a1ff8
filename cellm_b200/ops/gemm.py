from __future__ import annotations

import torch

from ._lib import check, fn, ptr, stream_of, tag


def gemm_plain(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T on the CUDA cores with 32-bit sums; rows may be strided."""
    if not (a.is_cuda and w.is_cuda) or a.stride(-1) != 1 or w.stride(-1) != 1:
        raise ValueError("gemm_plain: operands must be CUDA tensors with unit inner stride")
    if a.dtype != w.dtype or a.shape[1] != w.shape[1]:
        raise ValueError(f"gemm_plain: a {tuple(a.shape)} {a.dtype} and w {tuple(w.shape)} {w.dtype} do not fit")
    out_dtype = out_dtype or a.dtype
    M, K = a.shape
    N = w.shape[0]
    c = torch.empty((M, N), dtype=out_dtype, device=a.device)
    check(fn("gemm_plain", "cellm_gemm_plain")(ptr(c), ptr(a), ptr(w), M, N, K, a.stride(0), w.stride(0),
                                               c.stride(0), tag(a), tag(out_dtype), stream_of(a)), "gemm_plain")
    return c


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
         w_is_static: bool = False) -> torch.Tensor:
    """The product a . w^T by the kernel that serves the operands' element type:
    32-bit operands run the plain 32-bit kernel; bfloat16 operands run the
    tensor-core kernels."""
    if a.dtype == torch.float32:
        return gemm_plain(a, w, out_dtype)
    from .gemm_bf16 import gemm_bf16
    return gemm_bf16(a, w, out_dtype, w_is_static)
