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

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
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
             4: "state slot outside the pool", 8: "a bounded wait inside a kernel gave up",
             16: "shared memory not aligned as a kernel's tiles need"}


class StepRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, use_graphs: bool = False):
        self.model, self.cache = model, cache
        self.device = model.device
        self._forward = model.forward
        from ..ops._state import error_word
        self.err = error_word(self.device)      # one error word for every kernel on this device
        self._pinned = [None, None]
        self._events = [None, None]        # one reusable event per staging buffer: recorded after its upload
        self._recorded = [False, False]
        self._flip = 0
        self._layouts: dict = {}
        self.steps = 0
        self.tokens = 0
        self.use_graphs = use_graphs and model.graph_safe and self.device.type == "cuda"
        self.graph_width_step = 32        # block-table widths are rounded up to this many pages per graph
        # Captured decode steps by (entries, width bucket), least recently used first. Each holds its own logits
        # and activations (tens of MB at large batches), so a long-running engine keeps only the most recent ones.
        self._graphs: OrderedDict = OrderedDict()
        self.max_graphs = 128
        # A shape is captured when it is met for the capture_after-th time; until then its steps are launched kernel
        # by kernel. A capture costs several steps' time, and a batch that shrinks as requests end meets many shapes
        # once or twice.
        self.capture_after = 1
        self._met: dict = {}
        # arg-max of the last step's logits where the step's graph has computed it (greedy requests then
        # need no launch of their own); None after a step that ran without a graph
        self.last_argmax: Optional[torch.Tensor] = None
        # The tokens a captured decode step chose, by state slot of their requests: the step after it takes the ids it
        # was given as -1 from here (the engine may launch it before it has read this step's tokens).
        self.last_token = torch.zeros(max(cache.num_slots, 1), dtype=torch.int32, device=self.device)
        self._tok_host = [None, None]
        self._tok_events = [None, None]
        self._tok_flip = 0

    # ------------------------------------------------------------------
    def _staging(self, n: int) -> torch.Tensor:
        """A pinned int32 buffer of at least n values whose last upload has finished."""
        self._flip ^= 1
        i = self._flip
        if self._recorded[i]:
            self._events[i].synchronize()
        if self._pinned[i] is None or self._pinned[i].numel() < n:
            self._pinned[i] = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=True)
        return self._pinned[i]

    def _uploaded(self) -> None:
        """Marks the point in the stream after which the current staging buffer may be written again."""
        i = self._flip
        if self._events[i] is None:
            self._events[i] = torch.cuda.Event()
        self._events[i].record()
        self._recorded[i] = True

    def _prepare(self, entries: Sequence[StepEntry]):
        """Checks the entries and reserves their pages. Returns the host-side
        description of the batch: (q_lens, ctx_lens, slots, totals, token ids, logit rows)."""
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
        ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        V = self.model.plan.vocab_size
        if ids.min() < 0 or ids.max() >= V:
            raise ValueError(f"token id {int(ids.max() if ids.max() >= V else ids.min())} outside the vocabulary of {V}")
        cu = np.zeros(len(entries) + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu[1:])
        rows = [int(cu[b]) + w for b, e in enumerate(entries) for w in e.want]
        return q_lens, ctx_lens, slots, totals, ids, cu, rows

    def _fill(self, buf: np.ndarray, entries, q_lens, ctx_lens, slots, ids, cu, rows, width: int):
        """Writes the step's index arrays into `buf`; returns the (offset, length)
        of each array and the (offset, B, width) of each block table."""
        cache = self.cache
        B, T, R = len(entries), int(cu[-1]), len(rows)
        o = 0

        def put(arr, n):
            nonlocal o
            buf[o:o + n] = arr
            o += n
            return (o - n, n)
        spans = {"ids": put(ids, T),
                 "pos": put(np.concatenate([np.arange(c, c + n) for c, n in zip(ctx_lens, q_lens)]), T),
                 "seq": put(np.repeat(np.arange(B), q_lens), T),
                 "cu": put(cu, B + 1), "ctx": put(ctx_lens, B), "slot": put(slots, B),
                 "rows": put(rows, R) if R else (o, 0)}
        tables = []
        for g in range(len(cache.paged_keys)):
            tab = buf[o:o + B * width].reshape(B, width)
            tab.fill(-1)
            for b, e in enumerate(entries):
                cache.block_table(e.request_id, g, tab[b])
            tables.append((o, B, width))
            o += B * width
        return spans, tables, o

    def _meta_size(self, B, T, R, width) -> int:
        return 3 * T + (B + 1) + 2 * B + R + len(self.cache.paged_keys) * B * width

    def _context(self, dev: torch.Tensor, spans, tables, q_lens, ctx_lens, max_total_len):
        view = lambda s: dev[s[0]:s[0] + s[1]]
        T, B = spans["ids"][1], len(q_lens)
        ctx = StepContext(T=T, B=B, dtype=self.model.dtype, device=self.device, token_ids=view(spans["ids"]),
                          positions=view(spans["pos"]), seq_of_token=view(spans["seq"]), cu_seqlens=view(spans["cu"]),
                          ctx_lens=view(spans["ctx"]), slot_ids=view(spans["slot"]), err=self.err, q_lens=list(q_lens),
                          ctx_lens_host=list(ctx_lens), max_q_len=max(q_lens), max_total_len=max_total_len)
        tabs = [dev[o0:o0 + b * w].view(b, w) for (o0, b, w) in tables]
        logit_rows = view(spans["rows"]) if spans["rows"][1] else None
        return ctx, tabs, logit_rows

    def build_context(self, entries: Sequence[StepEntry]):
        """Checks the entries, reserves their pages and uploads the step's index
        arrays in one copy. Returns (ctx, block tables per paged group, logit rows, new totals)."""
        q_lens, ctx_lens, slots, totals, ids, cu, rows = self._prepare(entries)
        width = max((t + self.cache.page_size - 1) // self.cache.page_size for t in totals)
        n_meta = self._meta_size(len(entries), int(cu[-1]), len(rows), width)
        stage = self._staging(n_meta)
        spans, tables, n = self._fill(stage.numpy(), entries, q_lens, ctx_lens, slots, ids, cu, rows, width)
        dev = stage[:n_meta].to(self.device, non_blocking=True)
        self._uploaded()
        ctx, tabs, logit_rows = self._context(dev, spans, tables, q_lens, ctx_lens, max(totals))
        return ctx, tabs, logit_rows, totals

    # ------------------------------------------------------------- decoding with CUDA graphs
    def _run_decode_graph(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A step in which every entry is one token whose logits are wanted: the
        launches of such a step depend only on the number of entries and on the
        width of the block tables, so they are captured once per (entries, width
        bucket) in a CUDA graph and replayed; only the index arrays change."""
        q_lens, ctx_lens, slots, totals, ids, cu, rows = self._prepare(entries)
        B, ps = len(entries), self.cache.page_size
        need = max((t + ps - 1) // ps for t in totals)
        width = -(-need // self.graph_width_step) * self.graph_width_step
        n_meta = self._meta_size(B, B, B, width)
        stage = self._staging(n_meta)
        spans, tables, _ = self._fill(stage.numpy(), entries, q_lens, ctx_lens, slots, ids, cu, rows, width)
        g = self._graph_slot((B, width), n_meta)
        ops.upload(g["meta"], stage, n_meta)
        self._uploaded()
        if "graph" not in g:
            self._capture(g, spans, tables, q_lens, ctx_lens, width * ps, slots)
        from ..ops._lib import LAUNCHES
        g["graph"].replay()
        LAUNCHES[0] += g["launches"]
        for e, total in zip(entries, totals):
            self.cache.commit(e.request_id, total)
        self.steps += 1
        self.tokens += B
        self.last_argmax = g["argmax"]
        return g["logits"]

    def _ripe(self, key) -> bool:
        """Whether a decode step of this (entries, width bucket) is to be replayed as a graph (capturing it if need be)."""
        if key in self._graphs:
            return True
        n = self._met.get(key, 0) + 1
        if n >= self.capture_after:
            self._met.pop(key, None)
            return True
        if len(self._met) > 4096:
            self._met.clear()
        self._met[key] = n
        return False

    def _graph_slot(self, key, n_meta: int) -> dict:
        """The record of the captured step for `key`, made (and the least recently used one dropped) if need be."""
        g = self._graphs.get(key)
        if g is not None:
            self._graphs.move_to_end(key)
            return g
        if len(self._graphs) >= self.max_graphs:
            torch.cuda.synchronize(self.device)      # its last replay may still be running
            self._graphs.popitem(last=False)
        g = {"meta": torch.empty(n_meta, dtype=torch.int32, device=self.device)}
        self._graphs[key] = g
        return g

    def _layout(self, B: int, T: int, R: int, width: int):
        """Offsets of the index arrays for a step of this shape (the order `_fill` and
        the runtime's plan_fill write them in)."""
        o = 0
        spans = {}
        for name, n in (("ids", T), ("pos", T), ("seq", T), ("cu", B + 1), ("ctx", B), ("slot", B), ("rows", R)):
            spans[name] = (o, n)
            o += n
        tables = []
        for _ in range(len(self.cache.paged_keys)):
            tables.append((o, B, width))
            o += B * width
        return spans, tables, o

    def run_planned(self, scheduler, max_layers: Optional[int] = None) -> Optional[torch.Tensor]:
        """Runs the step the scheduler planned last. The runtime writes the index
        arrays itself (tokens, positions, slots, block tables), so the host's share of
        a step is a handful of calls whatever the batch. The scheduler has reserved
        the pages; its step_done() records the new lengths."""
        B, T, R, max_total, all_decode = scheduler.plan_shape()
        if B == 0:
            return None
        ps = self.cache.page_size
        need = (max_total + ps - 1) // ps
        graph = self.use_graphs and all_decode and max_layers is None
        graph = graph and self._ripe((B, -(-need // self.graph_width_step) * self.graph_width_step))
        width = -(-need // self.graph_width_step) * self.graph_width_step if graph else need
        lay = self._layouts.get((B, T, R, width))
        if lay is None:
            lay = self._layouts[(B, T, R, width)] = self._layout(B, T, R, width)
        spans, tables, n_meta = lay
        stage = self._staging(n_meta)
        scheduler.plan_fill(stage.data_ptr(), n_meta, width, len(self.cache.paged_keys))
        if all_decode:
            q_lens, ctx_lens = [1] * B, None
        else:
            buf = stage.numpy()
            cu = buf[spans["cu"][0]:spans["cu"][0] + B + 1]
            q_lens = np.diff(cu).tolist()
        self.steps += 1
        self.tokens += T
        if graph:
            g = self._graph_slot((B, width), n_meta)
            ops.upload(g["meta"], stage, n_meta)
            self._uploaded()
            if "graph" not in g:
                slots = stage.numpy()[spans["slot"][0]:spans["slot"][0] + B].tolist()
                self._capture(g, spans, tables, q_lens, [0] * B, width * ps, slots)
            from ..ops._lib import LAUNCHES
            g["graph"].replay()
            LAUNCHES[0] += g["launches"]
            self.last_argmax = g["argmax"]
            return g["logits"]
        self.last_argmax = None
        dev = stage[:n_meta].to(self.device, non_blocking=True)
        self._uploaded()
        ctx_lens = stage.numpy()[spans["ctx"][0]:spans["ctx"][0] + B].tolist()
        ctx, tabs, logit_rows = self._context(dev, spans, tables, q_lens, ctx_lens, max_total)
        if self.device.type == "cuda":
            ops.take_pending_tokens(ctx.token_ids, ctx.seq_of_token, ctx.slot_ids, self.last_token, self.err)
        return self._forward(ctx, self.cache.bindings(tabs), logit_rows, max_layers)

    def tokens_to_host(self):
        """Starts the copy of the last captured step's arg-max to pinned host memory; returns (pinned int32
        tensor, number of rows, event recorded after the copy). Two buffers take turns."""
        self._tok_flip ^= 1
        i = self._tok_flip
        n = self.last_argmax.numel()
        if self._tok_host[i] is None or self._tok_host[i].numel() < n:
            self._tok_host[i] = torch.empty(max(n, self.cache.num_slots, 64), dtype=torch.int32, pin_memory=True)
            self._tok_events[i] = torch.cuda.Event()
        self._tok_host[i][:n].copy_(self.last_argmax, non_blocking=True)
        self._tok_events[i].record()
        return self._tok_host[i], n, self._tok_events[i]

    def _capture(self, g: dict, spans, tables, q_lens, ctx_lens, max_total_len: int, slots) -> None:
        """Captures the forward pass over g["meta"] as a CUDA graph (see _run_decode_graph)."""
        from ..ops._lib import LAUNCHES
        ctx, tabs, logit_rows = self._context(g["meta"], spans, tables, q_lens, ctx_lens, max_total_len)
        bindings = self.cache.bindings(tabs)
        # One eager run loads every kernel this shape uses; fixed-size state is
        # put back afterwards, because the captured run will update it again.
        slot_idx = torch.tensor(slots, dtype=torch.long, device=self.device)
        saved = [s[:, slot_idx].clone() for s in self.cache.states]
        ops.take_pending_tokens(ctx.token_ids, ctx.seq_of_token, ctx.slot_ids, self.last_token, self.err)
        self.model.forward(ctx, bindings, logit_rows)
        for s, keep in zip(self.cache.states, saved):
            s[:, slot_idx] = keep
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = LAUNCHES[0]
        with torch.cuda.graph(graph):
            ops.take_pending_tokens(ctx.token_ids, ctx.seq_of_token, ctx.slot_ids, self.last_token, self.err)
            g["logits"] = self.model.forward(ctx, bindings, logit_rows)
            g["argmax"] = ops.argmax(g["logits"])          # greedy requests read their tokens here
            ops.keep_last_tokens(self.last_token, ctx.slot_ids, g["argmax"])
        g["graph"] = graph
        g["launches"] = LAUNCHES[0] - before     # kernels one replay runs
        LAUNCHES[0] = before

    def run(self, entries: Sequence[StepEntry], max_layers: Optional[int] = None) -> Optional[torch.Tensor]:
        """Runs one step; returns float32 logits [number of wanted places, vocab] in
        the order of the entries and of their `want`, or None if nothing is wanted.
        The tensor may be overwritten by the next step."""
        if self.use_graphs and max_layers is None and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            ps = self.cache.page_size
            need = max((self.cache.tokens(e.request_id) + ps) // ps for e in entries)      # pages of tokens + 1
            if self._ripe((len(entries), -(-need // self.graph_width_step) * self.graph_width_step)):
                return self._run_decode_graph(entries)
        self.last_argmax = None
        ctx, tables, logit_rows, totals = self.build_context(entries)
        logits = self._forward(ctx, self.cache.bindings(tables), logit_rows, max_layers)
        for e, total in zip(entries, totals):
            self.cache.commit(e.request_id, total)
        self.steps += 1
        self.tokens += ctx.T
        return logits

    def check_rarely(self, every: int = 64) -> None:
        """check() once in `every` calls: reading the error word back costs a
        round trip to the device, and a fault does not go away."""
        self._check_calls = getattr(self, "_check_calls", 0) + 1
        if self._check_calls % every == 1:
            self.check()

    def check(self) -> None:
        """Raises if a kernel flagged a fault since the last check (synchronises)."""
        code = int(self.err.item())
        if code:
            self.err.zero_()
            what = [msg for bit, msg in _ERR_BITS.items() if code & bit]
            raise DeviceFault("device error word set: " + "; ".join(what))
