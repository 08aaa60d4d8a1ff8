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


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """The product a [M, K] . w [N, K]^T by the kernel the native executor chooses for the operands: 32-bit
    operands run the plain 32-bit kernel; bfloat16 operands run the tensor-core kernel in the tile shape and K
    split that fit M, N and K (or the plain kernel where K or the rows' alignment do not fit it). `w` is taken
    for a weight that nothing on the stream writes."""
    from ..runtime import records as R
    from ..runtime.program import part_program
    if a.dtype != w.dtype or a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or a.stride(1) != 1 or w.stride(1) != 1:
        raise ValueError(f"gemm: a {tuple(a.shape)} {a.dtype} and w {tuple(w.shape)} {w.dtype} do not fit")
    out_dtype = out_dtype or a.dtype
    c = torch.empty((a.shape[0], w.shape[0]), dtype=out_dtype, device=a.device)
    if a.shape[0] == 0:
        return c
    rec = R.Record(R.LINEAR, R.LinearParams(R.linear(w), a.stride(0), tag(out_dtype)))
    if a.data_ptr() % 16:
        rec.params.w.tc_ok = 0
    part_program(a.dtype, a.device, a.shape[1]).run_part(rec, a, None, out=c, rows=a.shape[0])
    return c
