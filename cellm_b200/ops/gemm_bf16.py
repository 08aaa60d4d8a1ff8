"""bfloat16 matrix products on the tcgen05 tensor cores, with the choice of
tile shape and K split for the sizes at hand."""
from __future__ import annotations

import torch

from ._lib import LAUNCHES, check, fn, ptr, stream_of, tag
from .gemm import gemm_plain

_SM_COUNT: dict[int, int] = {}
_WORKSPACE: dict[torch.device, torch.Tensor] = {}
_ERR: dict[torch.device, torch.Tensor] = {}


def _sms(device) -> int:
    i = torch.device(device).index or 0
    if i not in _SM_COUNT:
        _SM_COUNT[i] = torch.cuda.get_device_properties(i).multi_processor_count
    return _SM_COUNT[i]


def _workspace(device, n_floats: int) -> torch.Tensor:
    if torch.cuda.is_current_stream_capturing():
        # a captured launch keeps its pointers: give it memory of the graph's own pool
        return torch.empty(n_floats, dtype=torch.float32, device=device)
    ws = _WORKSPACE.get(device)
    if ws is None or ws.numel() < n_floats:
        ws = torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=device)
        _WORKSPACE[device] = ws
    return ws


def error_word(device) -> torch.Tensor:
    """The device error word the tensor-core kernels report a timed-out wait in."""
    e = _ERR.get(device)
    if e is None:
        e = torch.zeros(1, dtype=torch.int32, device=device)
        _ERR[device] = e
    return e


def plan_tiles(M: int, N: int, K: int, sms: int) -> tuple[int, int]:
    """(bn, split_k) for a product of these sizes: bn > 0 plain tiles of 128 x bn,
    bn < 0 swapped tiles of 128 weight rows x -bn tokens."""
    kblocks = (K + 63) // 64
    if M <= 64:
        narrow = 16 if M <= 16 else (32 if M <= 32 else 64)
        tiles = (N + 127) // 128
        # enough CTAs to keep two per SM streaming, but at least four K blocks each
        split = max(1, min((2 * sms + tiles - 1) // tiles, kblocks // 4))
        return -narrow, split
    bn = 256 if N >= 256 else (128 if N > 64 else 64)
    tiles = ((N + bn - 1) // bn) * ((M + 127) // 128)
    split = 1
    if tiles < sms // 2:
        split = max(1, min(sms // tiles, kblocks // 4))
    return bn, split


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, bn: int, split_k: int,
                 err: torch.Tensor | None = None) -> torch.Tensor:
    M, K = a.shape
    N = w.shape[0]
    c = torch.empty((M, N), dtype=out_dtype, device=a.device)
    ws = _workspace(a.device, split_k * M * N) if split_k > 1 else None
    err = err if err is not None else error_word(a.device)
    check(fn("gemm_tcgen05", "cellm_gemm_tcgen05")(
        ptr(c), ptr(a), ptr(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), tag(out_dtype), int(bn),
        int(split_k), ptr(ws), ptr(err), stream_of(a)), "gemm_tcgen05")
    if split_k > 1:
        LAUNCHES[0] += 1
    return c


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """a [M, K] . w [N, K]^T for bfloat16 operands, 32-bit accumulation, output
    bfloat16 or float32. Sizes the tensor-core kernel does not take (K not a
    multiple of 8, unaligned rows) go to the plain kernel."""
    out_dtype = out_dtype or a.dtype
    M, K = a.shape
    if (K % 8) or a.stride(1) != 1 or w.stride(1) != 1 or (a.stride(0) % 8) or (w.stride(0) % 8) \
            or (a.data_ptr() % 16) or (w.data_ptr() % 16):
        return gemm_plain(a, w, out_dtype)
    bn, split = plan_tiles(M, w.shape[0], K, _sms(a.device))
    return gemm_tcgen05(a, w, out_dtype, bn, split)
