"""The step function: one batch of (request, its next tokens), portions of
prompts beside single decoded tokens, cut anywhere. It runs only the tokens it
is given, from the cache that earlier steps left, and returns the logits at
the wanted places.

The reference's step runs one token of one session
(crates/cellm-model/src/lfm.rs:263-270, with the position checks of :280-289);
its `prefill` is a loop over that (:230-249). Here the same precondition holds
per request — a portion starts where the request's cache ends — and all
portions of a step run as one batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages
from ..models.decoder import DecoderModel
from ..parts.base import StepContext


@dataclass
class StepEntry:
    request_id: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)   # places among `tokens` whose logits are wanted


class DeviceFault(RuntimeError):
    """A kernel reported a bad token id, page or slot through the device error word."""


_ERR_BITS = {1: "token id outside the vocabulary", 2: "page id outside the pool",
             4: "state slot outside the pool", 8: "a bounded wait inside a kernel gave up"}


class StepRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager):
        self.model, self.cache = model, cache
        self.device = model.device
        from ..ops.gemm_bf16 import error_word
        self.err = error_word(self.device)      # one error word for every kernel on this device
        self._pinned = [None, None]
        self._events = [None, None]
        self._flip = 0
        self.steps = 0
        self.tokens = 0

    # ------------------------------------------------------------------
    def _staging(self, n: int) -> torch.Tensor:
        """A pinned int32 buffer of at least n values whose last upload has finished."""
        self._flip ^= 1
        i = self._flip
        if self._events[i] is not None:
            self._events[i].synchronize()
        if self._pinned[i] is None or self._pinned[i].numel() < n:
            self._pinned[i] = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=True)
        return self._pinned[i]

    def build_context(self, entries: Sequence[StepEntry]):
        """Checks the entries, reserves their pages and uploads the step's index
        arrays in one copy. Returns (ctx, block tables per paged group, logit rows, new totals)."""
        cache = self.cache
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        q_lens, ctx_lens, slots, totals = [], [], [], []
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request_id}: an entry needs at least one token")
            if any(not 0 <= w < n for w in e.want):
                raise ValueError(f"request {e.request_id}: wanted places {list(e.want)} outside 0..{n - 1}")
            start = cache.tokens(e.request_id)
            if start + n > self.model.plan.max_positions:
                raise ValueError(f"request {e.request_id}: {start + n} tokens exceed the model's "
                                 f"{self.model.plan.max_positions} positions")
            q_lens.append(n)
            ctx_lens.append(start)
            slots.append(cache.slot(e.request_id))
            totals.append(start + n)
        for e, total in zip(entries, totals):
            if not cache.reserve(e.request_id, total):
                raise OutOfPages(f"request {e.request_id}: no pages left for {total} tokens "
                                 f"(free: {[cache.free_pages(g) for g in range(len(cache.paged_keys))]})")
        B, T = len(entries), sum(q_lens)
        ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        V = self.model.plan.vocab_size
        if ids.min() < 0 or ids.max() >= V:
            raise ValueError(f"token id {int(ids.max() if ids.max() >= V else ids.min())} outside the vocabulary of {V}")
        cu = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu[1:])
        rows = [int(cu[b]) + w for b, e in enumerate(entries) for w in e.want]
        R = len(rows)
        n_groups = len(cache.paged_keys)
        widths = [max((t + cache.page_size - 1) // cache.page_size for t in totals)] * n_groups
        n_meta = 3 * T + (B + 1) + 2 * B + R + sum(B * w for w in widths)
        stage = self._staging(n_meta)
        buf = stage.numpy()
        o = 0
        def put(arr, n):
            nonlocal o
            buf[o:o + n] = arr
            o += n
            return (o - n, n)
        s_ids = put(ids, T)
        s_pos = put(np.concatenate([np.arange(c, c + n) for c, n in zip(ctx_lens, q_lens)]), T)
        s_seq = put(np.repeat(np.arange(B), q_lens), T)
        s_cu = put(cu, B + 1)
        s_ctx = put(ctx_lens, B)
        s_slot = put(slots, B)
        s_rows = put(rows, R) if R else (o, 0)
        s_bt = []
        for g in range(n_groups):
            w = widths[g]
            tab = buf[o:o + B * w].reshape(B, w)
            tab.fill(-1)
            for b, e in enumerate(entries):
                cache.block_table(e.request_id, g, tab[b])
            s_bt.append((o, B, w))
            o += B * w
        dev = stage[:n_meta].to(self.device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[self._flip] = ev
        view = lambda s: dev[s[0]:s[0] + s[1]]
        ctx = StepContext(T=T, B=B, dtype=self.model.dtype, device=self.device, token_ids=view(s_ids),
                          positions=view(s_pos), seq_of_token=view(s_seq), cu_seqlens=view(s_cu),
                          ctx_lens=view(s_ctx), slot_ids=view(s_slot), err=self.err, q_lens=q_lens,
                          ctx_lens_host=ctx_lens, max_q_len=max(q_lens), max_total_len=max(totals))
        tables = [dev[o0:o0 + b * w].view(b, w) for (o0, b, w) in s_bt]
        logit_rows = view(s_rows) if R else None
        return ctx, tables, logit_rows, totals

    def run(self, entries: Sequence[StepEntry], max_layers: Optional[int] = None) -> Optional[torch.Tensor]:
        """Runs one step; returns float32 logits [number of wanted places, vocab] in
        the order of the entries and of their `want`, or None if nothing is wanted."""
        ctx, tables, logit_rows, totals = self.build_context(entries)
        logits = self.model.forward(ctx, self.cache.bindings(tables), logit_rows, max_layers)
        for e, total in zip(entries, totals):
            self.cache.commit(e.request_id, total)
        self.steps += 1
        self.tokens += ctx.T
        return logits

    def check(self) -> None:
        """Raises if a kernel flagged a fault since the last check (synchronises)."""
        code = int(self.err.item())
        if code:
            self.err.zero_()
            what = [msg for bit, msg in _ERR_BITS.items() if code & bit]
            raise DeviceFault("device error word set: " + "; ".join(what))
