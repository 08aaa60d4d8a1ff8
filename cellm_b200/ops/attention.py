from __future__ import annotations

import torch

from .basic import attention_plain


def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, ctx, block_table: torch.Tensor,
              nh: int, scale: float, window: int) -> torch.Tensor:
    """Attention of every token of the step over its request's pages. Chooses the
    kernel by element type and by the shape of the batch."""
    return attention_plain(q, k_pool, v_pool, ctx.positions, ctx.seq_of_token, block_table, nh, scale,
                           window, ctx.err)
