"""Interfaces of the parts a layer is put together from.

A part is built from its own parameters (`PartSpec.params`) and the tensors
the loader found for it. It never sees the model's configuration or name.

  Norm            forward(residual) -> normed activations
  Position        rotation(...) describes itself to a fused kernel, or apply(q, k, positions)
  Mixer           forward(x, ctx, cache) -> [T, hidden]; declares what cache it needs
  FeedForward     forward(x, ctx) -> [T, hidden]
  Block           forward(residual, ctx, cache): the arrangement of the above in a layer

Folding a norm into the products around it (optional; small batches in bfloat16).
A norm between two matrix products can give its sum of squares to the product before
it and its scale to the product after it, so that no norm kernel runs:
  - a block that knows which norm comes after a mixer or feed-forward offers it a
    `ResidualSink` in `ctx.sink`; a part that says `feeds_sink = True` hands the sink
    to its last `Linear`, which may add its output to the stream itself and return None;
  - the norm then returns a `Prescaled` instead of a tensor to a part that says
    `takes_prescaled = True`; that part hands it to its first `Linear`.
A part that says neither sees plain tensors, as before.

`weight_specs(params)` lists the tensors a part reads, with the shape each
must have in the file and the class of values a random model gives it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch


@dataclass(frozen=True)
class TensorSpec:
    shape: tuple[int, ...]
    init: str                    # "linear", "embedding", "norm", "conv_tap", "bias"
    optional: bool = False


# ---------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKV:
    """Keys and values that grow with the sequence, kept in pages.
    window = 0: all keys are kept; window = w: a token reads its last w keys."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class FixedState:
    """Per-request state of fixed size, zero at the request's start."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------------- step context
@dataclass
class StepContext:
    """What every part may know about the batch of one step.

    The batch is B entries (request portions) flattened to T tokens. Device
    tensors are int32. `ctx_lens` counts the tokens of each request that were
    in the cache before this step; a token's position is ctx_lens[b] + its
    index in the portion."""
    T: int
    B: int
    dtype: torch.dtype                  # activation dtype of this run
    device: torch.device
    token_ids: torch.Tensor             # [T]
    positions: torch.Tensor             # [T]
    seq_of_token: torch.Tensor          # [T] entry index of each token
    cu_seqlens: torch.Tensor            # [B+1]
    ctx_lens: torch.Tensor              # [B]
    slot_ids: torch.Tensor              # [B] state slot of each entry
    err: torch.Tensor                   # [1] device error word
    q_lens: list[int] = field(default_factory=list)      # host copies
    ctx_lens_host: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_total_len: int = 0
    extras: dict[str, Any] = field(default_factory=dict)  # per-step scratch shared between parts
    sink: Optional["ResidualSink"] = None                  # see "Folding a norm" above; set and cleared by the block

    @property
    def stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream


@dataclass
class CacheBinding:
    """The cache one item of the layer order works on in this step."""
    need: Any = None                          # PagedKV | FixedState | None
    writes: bool = True                       # False: the item reads another item's cache
    # paged
    k: Optional[torch.Tensor] = None          # [pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None  # [B, max_blocks] int32, -1 = no page
    page_size: int = 0
    num_pages: int = 0
    # fixed state
    state: Optional[torch.Tensor] = None      # [slots, *shape]
    num_slots: int = 0


@dataclass
class Prescaled:
    """A norm's output that is not formed: `u` is the stream times the norm's weight
    [T, dim], `parts` [T, n] partial sums of the stream's squares. The normed rows
    are u[t] / sqrt(sum(parts[t]) / dim + eps); `materialize()` forms them."""
    u: torch.Tensor
    parts: torch.Tensor
    dim: int
    eps: float
    materialize: Any


class ResidualSink:
    """An offer to a part's last product: add your output to this stream yourself,
    for the norm `norm` (an object with .weight, .eps, .dim) that comes next."""

    def __init__(self, residual: "Residual", norm):
        self.residual, self.norm = residual, norm

    def delivered(self, u: torch.Tensor, parts: torch.Tensor) -> None:
        self.residual.folded = (self.norm, u, parts)


class Residual:
    """The 32-bit residual stream with one pending addend.

    A mixer's or feed-forward's output is not added at once: it waits until the
    next norm, which adds and normalises in one kernel. `folded` is set instead
    when a product has already added its output (see ResidualSink)."""

    def __init__(self, x: torch.Tensor):
        assert x.dtype == torch.float32
        self.x = x
        self.pending: Optional[torch.Tensor] = None
        self.folded: Optional[tuple] = None      # (norm, u, parts) left by a product for exactly that norm

    def add(self, delta: Optional[torch.Tensor]) -> None:
        """delta None: the part has delivered its output through the sink."""
        if delta is None:
            return
        if self.pending is not None:
            self.flush()
        self.folded = None
        self.pending = delta

    def flush(self) -> torch.Tensor:
        from .. import ops
        if self.pending is not None:
            ops.residual_add(self.x, self.pending)
            self.pending = None
        return self.x


class Part:
    """Base of all parts: parameters in, tensors in."""
    kind: str = ""
    # True if forward() only launches work on the current stream (no host read of
    # device data, no host-side branching on it), so that a decode step may be
    # captured in a CUDA graph. A part that does not say so keeps its model eager.
    graph_safe: bool = False

    @classmethod
    def weight_specs(cls, params: dict) -> dict[str, TensorSpec]:
        return {}


class Norm(Part):
    def forward(self, residual: Residual, rows: Optional[torch.Tensor] = None, prescaled_ok: bool = False):
        """Adds the pending addend into the stream and returns the normed rows
        (all rows, or the given row indices without touching the stream). With
        `prescaled_ok` it may return a Prescaled when the product before has left one."""
        raise NotImplementedError

    def sink(self, residual: Residual, T: int) -> Optional[ResidualSink]:
        """A sink for the product before this norm, or None if this norm does not fold."""
        return None


class Position(Part):
    def rotation(self):
        """(rotary_dim, interleaved, inv_freq [rotary_dim/2, 2] float32 device tensor: high part, remainder) if the
        encoding is a rotation a fused kernel can apply, else None."""
        return None

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor):
        """Unfused form: returns (q, k) with the encoding applied. q: [T, heads, hd]."""
        raise NotImplementedError


class Mixer(Part):
    @classmethod
    def cache_need(cls, params: dict):
        """PagedKV, FixedState or None."""
        return None

    can_read_foreign_cache = False   # whether an order item may set cache_of for this mixer

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding, next_norm: Optional[Norm] = None) -> None:
        """`next_norm`: the norm that will read the stream after this block, if the caller knows it."""
        raise NotImplementedError

    def first_norm(self) -> Optional[Norm]:
        """The norm this block begins with (what a block before it may fold into)."""
        return None
