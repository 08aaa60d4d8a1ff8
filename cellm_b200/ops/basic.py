from __future__ import annotations

from typing import Optional

import torch

from ._lib import check, count_launch, fn, ptr, require_cuda, stream_of, tag

_LIB = "kernels_common"


def embed(table: torch.Tensor, ids: torch.Tensor, err: torch.Tensor) -> torch.Tensor:
    """Rows of `table` [V, H] for int32 ids [T] as float32 [T, H]."""
    require_cuda(table, ids, err)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    check(fn(_LIB, "cellm_embed")(ptr(out), ptr(table), tag(table), ptr(ids), T, H, V, ptr(err),
                                  stream_of(table)), "embed")
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                act_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [*, H] float32 (+= delta in place when rows is None); returns the normed
    rows in act_dtype: all of them, or those listed in `rows`."""
    require_cuda(x, delta, w, rows)
    H = x.shape[-1]
    if x.dtype != torch.float32 or w.numel() != H:
        raise ValueError("add_rmsnorm: x must be float32 [*, H] and w must have H values")
    if delta is not None and (delta.dtype != act_dtype or delta.shape != x.shape):
        raise ValueError(f"add_rmsnorm: delta {tuple(delta.shape)} {delta.dtype} does not match x {tuple(x.shape)} / {act_dtype}")
    n = x.shape[0] if rows is None else rows.numel()
    y = torch.empty((n, H), dtype=act_dtype, device=x.device)
    check(fn(_LIB, "cellm_add_rmsnorm")(ptr(x), ptr(delta), ptr(w), tag(w), ptr(y), ptr(rows), n, H,
                                        float(eps), tag(act_dtype), stream_of(x)), "add_rmsnorm")
    return y


def upload(dst: torch.Tensor, pinned: torch.Tensor, n: int) -> None:
    """The first n elements of a pinned host tensor into a device tensor of the same
    element type, asynchronously on the current stream."""
    if not dst.is_cuda or not pinned.is_pinned() or dst.dtype != pinned.dtype or n > dst.numel() or n > pinned.numel():
        raise ValueError("upload: a pinned host tensor into a device tensor of the same element type")
    code = fn(_LIB, "cellm_upload")(dst.data_ptr(), pinned.data_ptr(), n * dst.element_size(), stream_of(dst))
    if code != 0:
        raise RuntimeError(f"upload: CUDA error {code}")


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    require_cuda(x, delta)
    if x.dtype != torch.float32 or x.shape != delta.shape:
        raise ValueError("residual_add: x must be float32 and delta of the same shape")
    check(fn(_LIB, "cellm_residual_add")(ptr(x), ptr(delta), x.numel(), tag(delta), stream_of(x)), "residual_add")


def swiglu(gu: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """gu [T, 2*ff] = [gate | up] -> silu(gate) * up [T, ff] of `out_dtype` (default: gu's; float32 gate and up
    may give a bfloat16 result)."""
    require_cuda(gu)
    T, two_ff = gu.shape
    h = torch.empty((T, two_ff // 2), dtype=out_dtype or gu.dtype, device=gu.device)
    check(fn(_LIB, "cellm_swiglu")(ptr(h), ptr(gu), T, two_ff // 2, tag(h), tag(gu), stream_of(gu)), "swiglu")
    return h


def short_conv(bcx: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor,
               slot_ids: torch.Tensor, seq_of_token: torch.Tensor, cu_seqlens: torch.Tensor,
               err: torch.Tensor, max_q_len: int = 0) -> torch.Tensor:
    """bcx [T, 3H]; w [H, taps]; bias [H] or None; state [slots, taps-1, H] float32
    (read, then updated in place). Returns y [T, H]. `max_q_len`: the longest
    portion of the batch if the host knows it (0: unknown); short portions run a
    single fused kernel."""
    require_cuda(bcx, w, bias, state, slot_ids, seq_of_token, cu_seqlens, err)
    T, H3 = bcx.shape
    H, taps = w.shape
    if H3 != 3 * H or state.dtype != torch.float32 or tuple(state.shape[1:]) != (max(taps - 1, 0), H):
        raise ValueError(f"short_conv: shapes do not fit (bcx {tuple(bcx.shape)}, w {tuple(w.shape)}, state {tuple(state.shape)})")
    if bias is not None and (bias.dtype != w.dtype or bias.numel() != H):
        raise ValueError("short_conv: bias must have the taps' element type and H values")
    y = torch.empty((T, H), dtype=bcx.dtype, device=bcx.device)
    B = cu_seqlens.numel() - 1
    check(fn(_LIB, "cellm_short_conv")(ptr(y), ptr(bcx), ptr(w), ptr(bias), tag(w), ptr(state),
                                       state.stride(0), ptr(slot_ids), ptr(seq_of_token), ptr(cu_seqlens),
                                       T, B, H, taps, state.shape[0], int(max_q_len), tag(bcx), ptr(err),
                                       stream_of(bcx)), "short_conv")
    if taps > 1 and not 0 < max_q_len <= 4:
        count_launch()          # the state update is a launch of its own
    return y


def qk_norm_rope(qkv: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor], eps: float,
                 positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                 k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], page_size: int,
                 nh: int, nkv: int, hd: int, rot: int, interleaved: bool, inv_freq: Optional[torch.Tensor],
                 err: torch.Tensor) -> torch.Tensor:
    """qkv [T, (nh + 2*nkv)*hd] -> q [T, nh*hd] normed and rotated; keys (normed,
    rotated) and values written into the pools [pages, kv_heads, page_size, hd].
    nkv = 0: rows hold queries only and nothing is written."""
    require_cuda(q_w, k_w, positions, seq_of_token, block_table, k_pool, v_pool, inv_freq, err)
    if not qkv.is_cuda or qkv.stride(1) != 1:
        raise ValueError("qk_norm_rope: rows must lie on the GPU with unit inner stride")
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise ValueError(f"qk_norm_rope: row of {qkv.shape[1]} values, expected {(nh + 2 * nkv) * hd}")
    if rot > 0 and (inv_freq is None or inv_freq.dtype != torch.float32 or tuple(inv_freq.shape) != (rot // 2, 2)):
        raise ValueError("qk_norm_rope: inv_freq must be float32 [rot/2, 2] (high part, remainder)")
    if nkv > 0 and (k_pool.dtype != qkv.dtype or tuple(k_pool.shape[1:]) != (nkv, page_size, hd) or k_pool.shape != v_pool.shape):
        raise ValueError(f"qk_norm_rope: pool {tuple(k_pool.shape)} {k_pool.dtype} does not fit [pages, {nkv}, {page_size}, {hd}] {qkv.dtype}")
    w_tag = tag(q_w) if q_w is not None else 0
    q = torch.empty((T, nh * hd), dtype=qkv.dtype, device=qkv.device)
    check(fn(_LIB, "cellm_qk_norm_rope")(
        ptr(q), ptr(qkv), qkv.stride(0), ptr(q_w), ptr(k_w), w_tag, float(eps), ptr(positions),
        ptr(seq_of_token), ptr(block_table), block_table.stride(0) if block_table is not None else 0,
        ptr(k_pool), ptr(v_pool), k_pool.shape[0] if k_pool is not None else 0, page_size, T, nh, nkv, hd,
        rot, 1 if interleaved else 0, ptr(inv_freq), tag(qkv), ptr(err), stream_of(qkv)), "qk_norm_rope")
    return q


def attention_plain(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, positions: torch.Tensor,
                    seq_of_token: torch.Tensor, block_table: torch.Tensor, nh: int, scale: float,
                    window: int, err: torch.Tensor) -> torch.Tensor:
    """q [T, nh*hd]; pools [pages, kv_heads, page_size, hd]; each token reads keys
    0..positions[t] (or the last `window`) of its request."""
    require_cuda(q, k_pool, v_pool, positions, seq_of_token, block_table, err)
    pages, nkv, page_size, hd = k_pool.shape
    T = q.shape[0]
    if q.shape[1] != nh * hd or k_pool.dtype != q.dtype or v_pool.shape != k_pool.shape:
        raise ValueError("attention_plain: shapes or element types do not fit")
    out = torch.empty_like(q)
    check(fn(_LIB, "cellm_attention_plain")(
        ptr(out), ptr(q), ptr(k_pool), ptr(v_pool), ptr(positions), ptr(seq_of_token), ptr(block_table),
        block_table.stride(0), pages, page_size, T, nh, nkv, hd, float(scale), int(window), tag(q),
        ptr(err), stream_of(q)), "attention_plain")
    return out


def take_pending_tokens(ids: torch.Tensor, seq_of_token: torch.Tensor, slot_ids: torch.Tensor, last: torch.Tensor,
                        err: torch.Tensor) -> None:
    """Token ids of -1 (decoded tokens the host has not read yet) are replaced, in place, by last[state slot of the
    token's request], where the step before left them."""
    require_cuda(ids, seq_of_token, slot_ids, last, err)
    check(fn(_LIB, "cellm_take_pending_tokens")(ptr(ids), ptr(seq_of_token), ptr(slot_ids), ptr(last), ids.numel(),
                                                last.numel(), ptr(err), stream_of(ids)), "take_pending_tokens")


def keep_last_tokens(last: torch.Tensor, slot_ids: torch.Tensor, tokens: torch.Tensor) -> None:
    """last[slot_ids[r]] = tokens[r]: the tokens a decode step chose stay on the device for the step after it."""
    require_cuda(last, slot_ids, tokens)
    check(fn(_LIB, "cellm_keep_last_tokens")(ptr(last), ptr(slot_ids), ptr(tokens), tokens.numel(), last.numel(),
                                             stream_of(tokens)), "keep_last_tokens")


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Row-wise arg-max of float32 logits [R, V] as int32 [R]; lowest id among equals."""
    require_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise ValueError("argmax: logits must be float32 [R, V]")
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    # long rows are searched by 32 blocks each, which leave their finds in `parts` for a second, tiny kernel
    parts = torch.empty((R, 32), dtype=torch.int64, device=logits.device) if V >= 8192 else None
    check(fn(_LIB, "cellm_argmax")(ptr(out), ptr(logits), R, V, ptr(parts), stream_of(logits)), "argmax")
    if parts is not None:
        count_launch()
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, u: torch.Tensor,
           penalty: Optional[torch.Tensor] = None, recent: Optional[torch.Tensor] = None,
           max_top_k: int = 0, prefilter: bool = True) -> torch.Tensor:
    """One token per row of float32 logits [R, V]: arg-max where temperature <= 0,
    else a draw from softmax(logits / temperature) over the top_k logits (0: all),
    decided by the uniform number u[r]. recent [R, W] int32 (-1 padded) and
    penalty [R] apply the repetition penalty. max_top_k is the host's bound of top_k.
    `prefilter`: a first kernel finds the maxima of groups of 128 logits, which lets the
    rows that take a top k skip most of the row (off: one block searches the whole row;
    the choice is the same). Returns int32 [R]."""
    require_cuda(logits, temperature, top_k, u, penalty, recent)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise ValueError("sample: logits must be float32 [R, V]")
    R, V = logits.shape
    W = recent.shape[1] if recent is not None else 0
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    group_max = None
    if prefilter and 2048 <= V <= 128 * 8192:
        group_max = torch.empty((R, (V + 127) // 128), dtype=torch.int32, device=logits.device)
        count_launch()
    check(fn(_LIB, "cellm_sample")(ptr(out), ptr(logits), R, V, ptr(temperature), ptr(top_k), ptr(u),
                                   ptr(penalty), ptr(recent), W, int(max_top_k), ptr(group_max),
                                   stream_of(logits)), "sample")
    return out
