from __future__ import annotations

import torch

from ._lib import check, count_launch, fn, ptr, require_cuda, stream_of
from .basic import attention_plain

_FLASH_HEAD_SIZES = (32, 64, 128)
_WORKSPACE: dict[torch.device, torch.Tensor] = {}


def _workspace(device, n_floats: int) -> torch.Tensor:
    if torch.cuda.is_current_stream_capturing():
        # a captured launch keeps its pointers: give it memory of the graph's own pool
        return torch.empty(n_floats, dtype=torch.float32, device=device)
    ws = _WORKSPACE.get(device)
    if ws is None or ws.numel() < n_floats:
        ws = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
        _WORKSPACE[device] = ws
    return ws


def attention_flash(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, cu_seqlens: torch.Tensor,
                    ctx_lens: torch.Tensor, block_table: torch.Tensor, q_lens: list[int], nh: int, scale: float,
                    window: int, err: torch.Tensor, nsplit: int = 1, wide: bool | None = None) -> torch.Tensor:
    """Tensor-core attention for bfloat16: q [T, nh*hd], pools [pages, kv heads,
    page size, hd]; request b owns tokens cu_seqlens[b]..cu_seqlens[b+1] at
    positions ctx_lens[b] + i. `q_lens` are the host's copies of the portions' lengths."""
    require_cuda(q, k_pool, v_pool, cu_seqlens, ctx_lens, block_table, err)
    pages, nkv, page_size, hd = k_pool.shape
    T, B = q.shape[0], len(q_lens)
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or q.shape[1] != nh * hd or hd not in _FLASH_HEAD_SIZES:
        raise ValueError("attention_flash: bfloat16 with head size 32, 64 or 128 only")
    G = nh // nkv
    if wide is None:
        wide = max(q_lens) * G > 16
    bm = 64 if wide else 16
    n_tiles = sum((n * G + bm - 1) // bm for n in q_lens)
    out = torch.empty_like(q)
    part_o = part_ml = None
    if nsplit > 1:
        rows = T * nh
        ws = _workspace(q.device, nsplit * rows * (hd + 2))
        part_o, part_ml = ws[:nsplit * rows * hd], ws[nsplit * rows * hd:nsplit * rows * (hd + 2)]
    check(fn("attention_flash", "cellm_attention_flash")(
        ptr(out), ptr(part_o), ptr(part_ml), ptr(q), ptr(k_pool), ptr(v_pool), ptr(cu_seqlens), ptr(ctx_lens),
        ptr(block_table), block_table.stride(0), B, T, n_tiles, pages, page_size, nh, nkv, hd, float(scale),
        int(window), 1 if wide else 0, int(nsplit), ptr(err), stream_of(q)), "attention_flash")
    if nsplit > 1:
        count_launch()
    return out


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, cu_seqlens: torch.Tensor,
                     ctx_lens: torch.Tensor, block_table: torch.Tensor, B: int, nh: int, scale: float, window: int,
                     err: torch.Tensor, nsplit: int = 1) -> torch.Tensor:
    """Tensor-core attention for short portions (decoded tokens): every request has
    at most 16 / (nh / kv heads) tokens in the step. One CTA per (request, kv head,
    piece of the keys). Up to 8 pieces are one thread-block cluster and are combined through its shared memory; more
    go through a workspace, and the last CTA of a request to finish combines them."""
    require_cuda(q, k_pool, v_pool, cu_seqlens, ctx_lens, block_table, err)
    pages, nkv, page_size, hd = k_pool.shape
    T = q.shape[0]
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or q.shape[1] != nh * hd or hd not in _FLASH_HEAD_SIZES:
        raise ValueError("attention_decode: bfloat16 with head size 32, 64 or 128 only")
    out = torch.empty_like(q)
    part_o = part_ml = counters = None
    if nsplit > 8:
        from ._state import MAX_COUNTERS, counters as _counters
        if B * nkv > MAX_COUNTERS:
            raise ValueError("attention_decode: too many (request, kv head) pairs for the counters")
        rows = T * nh
        ws = _workspace(q.device, nsplit * rows * (hd + 2))
        part_o, part_ml = ws[:nsplit * rows * hd], ws[nsplit * rows * hd:nsplit * rows * (hd + 2)]
        counters = _counters(q.device)
    check(fn("attention_decode", "cellm_attention_decode")(
        ptr(out), ptr(part_o), ptr(part_ml), ptr(counters), ptr(q), ptr(k_pool), ptr(v_pool), ptr(cu_seqlens),
        ptr(ctx_lens), ptr(block_table), block_table.stride(0), B, T, pages, page_size, nh, nkv, hd, float(scale),
        int(window), int(nsplit), ptr(err), stream_of(q)), "attention_decode")
    return out


def attention_tc_supports(hd: int, nh: int, nkv: int, page_size: int) -> bool:
    """Sizes the tcgen05 prompt kernel takes: heads of 64, a group size that divides 128,
    pages of 8 to 128 tokens (powers of two)."""
    if hd != 64 or nkv <= 0 or nh % nkv:
        return False
    g = nh // nkv
    return g <= 128 and 128 % g == 0 and page_size in (8, 16, 32, 64, 128)


def attention_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, cu_seqlens: torch.Tensor,
                 ctx_lens: torch.Tensor, block_table: torch.Tensor, q_lens: list[int], nh: int, scale: float,
                 window: int, err: torch.Tensor) -> torch.Tensor:
    """Attention for prompt portions on the tcgen05 tensor cores (scores and outputs in
    tensor memory): bfloat16, heads of 64; arguments as attention_flash."""
    require_cuda(q, k_pool, v_pool, cu_seqlens, ctx_lens, block_table, err)
    pages, nkv, page_size, hd = k_pool.shape
    if q.dtype != torch.bfloat16 or k_pool.dtype != torch.bfloat16 or q.shape[1] != nh * hd \
            or not attention_tc_supports(hd, nh, nkv, page_size) or scale <= 0:
        raise ValueError("attention_tc: bfloat16, heads of 64, a group size dividing 128, pages of 8..128 tokens")
    tok_per_cta = 256 // (nh // nkv)             # a CTA takes two tiles of 128 (token, head) rows
    n_tiles = sum((n + tok_per_cta - 1) // tok_per_cta for n in q_lens)
    out = torch.empty_like(q)
    check(fn("attention_tc", "cellm_attention_tc")(
        ptr(out), ptr(q), ptr(k_pool), ptr(v_pool), ptr(cu_seqlens), ptr(ctx_lens), ptr(block_table),
        block_table.stride(0), len(q_lens), q.shape[0], n_tiles, pages, page_size, nh, nkv, hd, float(scale),
        int(window), ptr(err), stream_of(q)), "attention_tc")
    return out


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, block_table: torch.Tensor,
              nh: int, scale: float, window: int) -> torch.Tensor:
    """Attention of every token of the step over its request's pages, by the kernel the native executor chooses:
    bfloat16 with a head size the tensor-core kernels are built for runs there (decoded tokens in the decode
    kernel, large batches of prompt tokens with heads of 64 on tcgen05, the rest on mma.sync); everything else
    (32-bit, other head sizes) runs the plain kernel. q [T, nh * hd] (normed, turned) -> [T, nh * hd]."""
    from ..parts.base import CacheBinding
    from ..runtime import records as R
    from ..runtime.program import part_program
    pages, nkv, page_size, hd = k_pool.shape
    p = R.AttentionParams()
    p.nh, p.nkv, p.hd, p.window, p.scale = nh, nkv, hd, int(window), float(scale)
    out = torch.empty_like(q)
    binding = CacheBinding(k=k_pool, v=v_pool, block_table=block_table, page_size=page_size, num_pages=pages)
    part_program(q.dtype, q.device, q.shape[1]).run_part(R.Record(R.ATTEND, p), q, ctx, binding, out=out)
    return out
