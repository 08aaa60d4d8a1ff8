"""bfloat16 matrix products on the tcgen05 tensor cores, with the choice of
tile shape and K split for the sizes at hand."""
from __future__ import annotations

import functools

import torch

from ._lib import check, count_launch, fn, ptr, stream_of, tag
from .gemm import gemm_plain

from ._state import MAX_COUNTERS, STATIC_WEIGHTS_FLAG as _STATIC_FLAG, counters as _counters, error_word, sm_count as _sms

_WORKSPACE: dict[torch.device, torch.Tensor] = {}


def _workspace(device, n_floats: int) -> torch.Tensor:
    if torch.cuda.is_current_stream_capturing():
        # a captured launch keeps its pointers: give it memory of the graph's own pool
        return torch.empty(n_floats, dtype=torch.float32, device=device)
    ws = _WORKSPACE.get(device)
    if ws is None or ws.numel() < n_floats:
        ws = torch.empty(max(n_floats, 1 << 22), dtype=torch.float32, device=device)
        _WORKSPACE[device] = ws
    return ws


@functools.lru_cache(maxsize=4096)
def plan_tiles(M: int, N: int, K: int, sms: int) -> tuple[int, int]:
    """(bn, split_k) for a product of these sizes, as the native executor plans it: bn > 0 plain tiles of
    128 x bn, bn < 0 swapped tiles of 128 weight rows x -bn tokens."""
    from ..runtime.program import plan_tiles as planned
    return planned(M, N, K, sms)


@functools.lru_cache(maxsize=4096)
def _effective_split(K: int, split_k: int) -> int:
    kblocks = (K + 63) // 64
    split_k = max(1, min(split_k, kblocks))
    per = (kblocks + split_k - 1) // split_k
    return (kblocks + per - 1) // per


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, bn: int, split_k: int,
                 err: torch.Tensor | None = None, epilogue: int = 0, w_is_static: bool = False) -> torch.Tensor:
    """The tensor-core kernel with a given tile shape and split. epilogue 1: `w`
    holds blocks of 64 gate rows followed by their 64 up rows and the result is
    silu(gate) * up, [M, N/2]."""
    M, K = a.shape
    N = w.shape[0]
    c = torch.empty((M, N // 2 if epilogue else N), dtype=out_dtype, device=a.device)
    split = _effective_split(K, split_k)
    # swapped tiles whose K split is one thread-block cluster (2..8 CTAs) sum their pieces
    # through shared memory: no workspace, no counters
    in_cluster = bn < 0 and (2 <= split <= 8 or (split == 1 and epilogue == 1))
    through_ws = not in_cluster and (split > 1 or (epilogue == 1 and bn < 0))
    ws = _workspace(a.device, split * M * N) if through_ws else None
    # plain tiles leave the sum of their K-split pieces to a second kernel (no counters); swapped tiles outside a
    # cluster let the last CTA of a tile sum them
    counters = _counters(a.device) if (split > 1 and not in_cluster and bn < 0) else None
    err = err if err is not None else error_word(a.device)
    check(fn("gemm_tcgen05", "cellm_gemm_tcgen05")(
        ptr(c), ptr(a), ptr(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), tag(out_dtype), int(bn),
        int(split_k), int(epilogue), _STATIC_FLAG if w_is_static else 0, ptr(ws), ptr(counters), ptr(err), stream_of(a)),
        "gemm_tcgen05")
    if bn > 0 and split > 1:
        count_launch()          # the kernel that sums the K-split pieces
    return c


def tensor_core_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    K = a.shape[1]
    return not ((K % 8) or a.stride(1) != 1 or w.stride(1) != 1 or (a.stride(0) % 8) or (w.stride(0) % 8)
                or (a.data_ptr() % 16) or (w.data_ptr() % 16))


def gemm_swiglu_bf16(a: torch.Tensor, w_blocked: torch.Tensor, w_is_static: bool = False) -> torch.Tensor:
    """silu(a . w1^T) * (a . w3^T) in one kernel; `w_blocked` is w1 and w3 cut into
    blocks of 64 rows and laid out gate block, up block, gate block, ...; the
    caller has checked `tensor_core_ok` and that the width is a multiple of 64."""
    bn, split = plan_tiles(a.shape[0], w_blocked.shape[0], a.shape[1], _sms(a.device))
    if bn == 64:
        bn = 128
    return gemm_tcgen05(a, w_blocked, a.dtype, bn, split, epilogue=1, w_is_static=w_is_static)


CONV_TILE_CHANNELS = 42     # channels whose B, C and x rows share a tile of 128 rows
CONV_MAX_TAPS = 4


def tile_in_proj_for_conv(in_proj: torch.Tensor) -> torch.Tensor:
    """in_proj [3H, K] (B rows, C rows, x rows) cut into tiles of 128 rows that hold, for 42
    channels each, the 42 B rows, the 42 C rows and the 42 x rows (rows of channels beyond H and
    the last two rows of a tile are zero): the layout `gemm_conv_bf16` reads."""
    H3, K = in_proj.shape
    H, ch = H3 // 3, CONV_TILE_CHANNELS
    tiles = (H + ch - 1) // ch
    parts = in_proj.reshape(3, H, K)
    padded = torch.zeros((3, tiles * ch, K), dtype=in_proj.dtype, device=in_proj.device)
    padded[:, :H] = parts
    out = torch.zeros((tiles, 128, K), dtype=in_proj.dtype, device=in_proj.device)
    out[:, :3 * ch] = padded.reshape(3, tiles, ch, K).permute(1, 0, 2, 3).reshape(tiles, 3 * ch, K)
    return out.reshape(tiles * 128, K).contiguous()


def gemm_conv_plan(M: int, H: int, K: int, device) -> tuple[int, int] | None:
    """(bn, split_k) for the product with the convolution in its epilogue, or None if these
    sizes do not run it (it needs swapped tiles whose K split is one cluster)."""
    tiles = (H + CONV_TILE_CHANNELS - 1) // CONV_TILE_CHANNELS
    bn, split = plan_tiles(M, tiles * 128, K, _sms(device))
    if bn >= 0 or (M + -bn - 1) // -bn != 1 or _effective_split(K, split) > 8:
        return None
    return bn, split


def gemm_conv_bf16(a: torch.Tensor, w_tiled: torch.Tensor, H: int, taps: torch.Tensor, bias: torch.Tensor | None,
                   state: torch.Tensor, slot_ids: torch.Tensor, plan: tuple[int, int],
                   err: torch.Tensor | None = None) -> torch.Tensor:
    """One token of each of M requests: y [M, H] = C * conv(B * x) with B | C | x = a . in_proj^T, the
    convolution's history read from and moved on in `state` [slots, taps-1, H] (float32) at each
    request's slot. `w_tiled` is in_proj as `tile_in_proj_for_conv` lays it out; `plan` comes from
    `gemm_conv_plan`. The arithmetic is that of the product followed by `short_conv`."""
    M, K = a.shape
    n_taps = taps.shape[1]
    if a.dtype != torch.bfloat16 or w_tiled.dtype != torch.bfloat16 or taps.dtype != torch.bfloat16 \
            or (bias is not None and bias.dtype != torch.bfloat16) or state.dtype != torch.float32:
        raise ValueError("gemm_conv_bf16: bfloat16 activations, weights and taps, float32 state")
    if tuple(state.shape[1:]) != (n_taps - 1, H) or taps.shape[0] != H or slot_ids.numel() != M:
        raise ValueError(f"gemm_conv_bf16: shapes do not fit (state {tuple(state.shape)}, taps {tuple(taps.shape)}, {M} tokens)")
    y = torch.empty((M, H), dtype=torch.bfloat16, device=a.device)
    err = err if err is not None else error_word(a.device)
    check(fn("gemm_tcgen05", "cellm_gemm_conv_tcgen05")(
        ptr(y), ptr(a), ptr(w_tiled), M, w_tiled.shape[0], K, a.stride(0), w_tiled.stride(0), H, int(plan[0]), int(plan[1]),
        ptr(taps), ptr(bias), n_taps, ptr(state), state.stride(0), ptr(slot_ids), state.shape[0], _STATIC_FLAG,
        ptr(err), stream_of(a)), "gemm_conv_tcgen05")
    return y


def gemm_rope_plan(M: int, nh: int, nkv: int, hd: int, K: int, device) -> tuple[int, int] | None:
    """(bn, split_k) for the q/k/v product with norm, rotation and cache write in its epilogue, or
    None if these sizes do not run it (heads of 64; swapped tiles whose K split is one cluster)."""
    if hd != 64:
        return None
    bn, split = plan_tiles(M, (nh + 2 * nkv) * hd, K, _sms(device))
    if bn >= 0 or (M + -bn - 1) // -bn != 1 or _effective_split(K, split) > 8:
        return None
    return bn, split


def gemm_rope_bf16(a: torch.Tensor, w_qkv: torch.Tensor, q_w: torch.Tensor, k_w: torch.Tensor, eps: float,
                   positions: torch.Tensor, block_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   nh: int, nkv: int, inv_freq: torch.Tensor, plan: tuple[int, int],
                   err: torch.Tensor | None = None) -> torch.Tensor:
    """One token of each of M requests: q [M, nh * 64], normed and turned, from a . w_qkv^T; the keys (normed,
    turned) and values go to the requests' pages [pages, kv heads, page_size, 64]. Heads of 64 turned whole in
    pairs (i, i + 32); `plan` comes from `gemm_rope_plan`. The arithmetic is that of the product followed by
    `qk_norm_rope`."""
    M, K = a.shape
    pages, pool_kv, page_size, hd = k_pool.shape
    bf = torch.bfloat16
    if a.dtype != bf or w_qkv.dtype != bf or q_w.dtype != bf or k_w.dtype != bf or k_pool.dtype != bf or v_pool.dtype != bf:
        raise ValueError("gemm_rope_bf16: bfloat16 activations, weights, norm weights and pools")
    if hd != 64 or pool_kv != nkv or v_pool.shape != k_pool.shape or w_qkv.shape[0] != (nh + 2 * nkv) * 64 \
            or q_w.numel() != 64 or k_w.numel() != 64 or tuple(inv_freq.shape) != (32, 2) or inv_freq.dtype != torch.float32 \
            or positions.numel() != M or block_table.shape[0] != M:
        raise ValueError("gemm_rope_bf16: shapes do not fit (heads of 64, one block-table row and one position per token)")
    q = torch.empty((M, nh * 64), dtype=bf, device=a.device)
    err = err if err is not None else error_word(a.device)
    check(fn("gemm_tcgen05", "cellm_gemm_rope_tcgen05")(
        ptr(q), ptr(a), ptr(w_qkv), M, K, a.stride(0), w_qkv.stride(0), int(plan[0]), int(plan[1]), ptr(q_w), ptr(k_w),
        float(eps), ptr(positions), ptr(block_table), block_table.stride(0), ptr(k_pool), ptr(v_pool), pages, page_size,
        nh, nkv, ptr(inv_freq), _STATIC_FLAG, ptr(err), stream_of(a)), "gemm_rope_tcgen05")
    return q
