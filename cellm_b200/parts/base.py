"""Interfaces of the parts a layer is put together from.

A part is built from its own parameters (`PartSpec.params`) and the tensors
the loader found for it. It never sees the model's configuration or name.

  Embedding       forward(token_ids, ctx) -> the 32-bit residual stream [T, hidden]
  Norm            forward(residual) -> normed activations
  Position        rotation(...) describes itself to a fused kernel, or apply(q, k, positions)
  Mixer           forward(x, ctx, cache) -> [T, hidden]; declares what cache it needs
  FeedForward     forward(x, ctx) -> [T, hidden]
  Block           forward(residual, ctx, cache): the arrangement of the above in a layer
  Head            forward(x) -> float32 logits [rows, vocab]

`weight_specs(params)` lists the tensors a part reads, with the shape each
must have in the file and the class of values a random model gives it.

`emit(emitter)` describes the part to the native executor
(cellm_b200/runtime): a built-in part appends its own op record
(`emitter.native(kind, params)`), and the defaults below append a Python
record, for which the executor calls the part's forward() on its registers. So
a part defined outside the package needs forward() only, and runs between
native parts without slowing them.
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


class Residual:
    """The 32-bit residual stream with one pending addend.

    A mixer's or feed-forward's output is not added at once: it waits until the
    next norm, which adds and normalises in one kernel."""

    def __init__(self, x: torch.Tensor):
        assert x.dtype == torch.float32
        self.x = x
        self.pending: Optional[torch.Tensor] = None

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            self.flush()
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


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor, ctx: "StepContext") -> torch.Tensor:
        """The start of the residual stream: float32 [T, hidden]."""
        raise NotImplementedError

    def emit(self, emitter) -> None:
        emitter.python("embedding", self)


class Head(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """float32 logits [rows, vocab] of the normed rows x [rows, hidden]."""
        raise NotImplementedError

    def emit(self, emitter) -> None:
        emitter.python("head", self)


class Norm(Part):
    def emit(self, emitter) -> None:
        emitter.python("norm", self)

    def forward(self, residual: Residual, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Adds the pending addend into the stream and returns the normed rows
        (all rows, or the given row indices without touching the stream)."""
        raise NotImplementedError


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

    def emit(self, emitter) -> None:
        emitter.python("mixer", self)


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def emit(self, emitter) -> None:
        emitter.python("feed_forward", self)


class Block(Part):
    def forward(self, residual: Residual, ctx: StepContext, cache: CacheBinding) -> None:
        raise NotImplementedError

    def emit(self, emitter) -> None:
        emitter.python("block", self)
