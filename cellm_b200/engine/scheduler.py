"""Python face of the native scheduler (csrc/runtime/scheduler.cc)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from ..cache.manager import CacheManager
from ..cache.native import checked, int_array, last_error, lib


class SchedulerError(RuntimeError):
    pass


@dataclass
class PlannedEntry:
    request_id: int
    start: int
    count: int
    wants_logits: bool


@dataclass
class StepPlan:
    entries: list[PlannedEntry]
    preempted: list[int]
    admitted: list[tuple[int, int]]      # (request, state slot)


STATES = ("waiting", "prefill", "decoding", "finished")


class Scheduler:
    """Admits requests, cuts prompts into portions under a token budget, lets all
    decoding requests take one token per step, finishes and frees. When pages
    run out the most recently admitted running request is preempted and later
    recomputed from its prompt and the tokens generated so far."""

    def __init__(self, cache: CacheManager, max_batch_tokens: int, prefill_chunk: int, max_positions: int):
        self.cache = cache
        self._h = lib().cellm_sched_create(cache.handle, int(max_batch_tokens), int(prefill_chunk), int(max_positions))
        if not self._h:
            raise SchedulerError(last_error())
        self._cap = max(int(max_batch_tokens), cache.num_slots) + 8
        self._ids = (ctypes.c_longlong * self._cap)()
        self._a = (ctypes.c_int * self._cap)()
        self._b = (ctypes.c_int * self._cap)()
        self._c = (ctypes.c_int * self._cap)()

    def __del__(self):
        if getattr(self, "_h", None):
            lib().cellm_sched_destroy(self._h)
            self._h = None

    def add_request(self, request_id: int, tokens, max_new: int) -> None:
        checked(lib().cellm_sched_add(self._h, int(request_id), int_array(list(tokens)), len(tokens), int(max_new)),
                SchedulerError)

    def schedule(self) -> StepPlan:
        l = lib()
        checked(l.cellm_sched_schedule(self._h), SchedulerError)
        n = checked(l.cellm_sched_plan_entries(self._h, self._ids, self._a, self._b, self._c, self._cap), SchedulerError)
        entries = [PlannedEntry(self._ids[i], self._a[i], self._b[i], bool(self._c[i])) for i in range(n)]
        n = checked(l.cellm_sched_plan_preempted(self._h, self._ids, self._cap), SchedulerError)
        preempted = [self._ids[i] for i in range(n)]
        n = checked(l.cellm_sched_plan_admitted(self._h, self._ids, self._a, self._cap), SchedulerError)
        admitted = [(self._ids[i], self._a[i]) for i in range(n)]
        return StepPlan(entries, preempted, admitted)

    def plan_shape(self) -> tuple[int, int, int, int, bool]:
        """(entries, tokens, wanted rows, most tokens of a request after the step, all
        entries are single decoded tokens) of the step planned last."""
        buf = (ctypes.c_int * 5)()
        lib().cellm_sched_plan_shape(self._h, buf)
        return buf[0], buf[1], buf[2], buf[3], bool(buf[4])

    def plan_fill(self, buf_address: int, capacity: int, width: int, n_groups: int) -> int:
        """Has the runtime write the planned step's index arrays (ids, positions,
        entry of token, cumulative lengths, cached lengths, slots, wanted rows, block
        tables) straight into an int32 buffer; returns how many ints were written."""
        return checked(lib().cellm_sched_plan_fill(self._h, buf_address, int(capacity), int(width), int(n_groups)),
                       SchedulerError)

    def append_rows(self, tokens, stops) -> list[bool]:
        """One sampled token per wanted row of the planned step; returns which requests finished."""
        n = len(tokens)
        fin = (ctypes.c_int * max(n, 1))()
        checked(lib().cellm_sched_append_rows(self._h, int_array(list(tokens)), int_array([1 if x else 0 for x in stops]),
                                              fin, n), SchedulerError)
        return [bool(fin[i]) for i in range(n)]

    PENDING_TOKEN = -1

    def append_pending_rows(self, n: int) -> list[bool]:
        """One token per wanted row of the planned step whose value is not known yet (its step still runs);
        returns which requests have all their tokens with it."""
        return self.append_rows([self.PENDING_TOKEN] * n, [False] * n)

    def resolve_rows(self, request_ids, indices, tokens, stops) -> list[bool]:
        """The values of pending tokens (request, place among the request's tokens, value, whether it ends the
        request); returns which requests are finished (or gone) afterwards."""
        n = len(tokens)
        fin = (ctypes.c_int * max(n, 1))()
        ids = (ctypes.c_longlong * max(n, 1))(*[int(r) for r in request_ids])
        checked(lib().cellm_sched_resolve_rows(self._h, ids, int_array(list(indices)), int_array(list(tokens)),
                                               int_array([1 if x else 0 for x in stops]), fin, n), SchedulerError)
        return [bool(fin[i]) for i in range(n)]

    def schedule_rows(self):
        """Plans the next step like schedule(), but returns only what the engine needs
        per step: (ids of the requests whose logits are wanted, in row order;
        preempted requests; newly admitted (request, slot) pairs; number of entries)."""
        l = lib()
        n_entries = checked(l.cellm_sched_schedule(self._h), SchedulerError)
        n = checked(l.cellm_sched_plan_entries(self._h, self._ids, self._a, self._b, self._c, self._cap), SchedulerError)
        rows = [self._ids[i] for i in range(n) if self._c[i]]
        n = checked(l.cellm_sched_plan_preempted(self._h, self._ids, self._cap), SchedulerError)
        preempted = [self._ids[i] for i in range(n)] if n else []
        n = checked(l.cellm_sched_plan_admitted(self._h, self._ids, self._a, self._cap), SchedulerError)
        admitted = [(self._ids[i], self._a[i]) for i in range(n)] if n else []
        return rows, preempted, admitted, n_entries

    def step_done(self) -> None:
        """Marks the tokens of the last planned step as cached."""
        checked(lib().cellm_sched_step_done(self._h), SchedulerError)

    def append_token(self, request_id: int, token: int, stop: bool = False) -> bool:
        """Adds a sampled token; True when the request is finished (and freed)."""
        return bool(checked(lib().cellm_sched_append(self._h, int(request_id), int(token), 1 if stop else 0),
                            SchedulerError))

    def cancel(self, request_id: int) -> None:
        checked(lib().cellm_sched_cancel(self._h, int(request_id)), SchedulerError)

    def forget(self, request_id: int) -> None:
        checked(lib().cellm_sched_forget(self._h, int(request_id)), SchedulerError)

    def has(self, request_id: int) -> bool:
        return bool(lib().cellm_sched_has(self._h, int(request_id)))

    def info(self, request_id: int) -> dict:
        buf = (ctypes.c_int * 6)()
        checked(lib().cellm_sched_info(self._h, int(request_id), buf), SchedulerError)
        return {"state": STATES[buf[0]], "prompt_len": buf[1], "num_tokens": buf[2], "computed": buf[3],
                "generated": buf[4], "preemptions": buf[5],
                "finish_reason": lib().cellm_sched_finish_reason(self._h, int(request_id)).decode()}

    def tokens(self, request_id: int, start: int = 0, count: int | None = None) -> list[int]:
        total = self.info(request_id)["num_tokens"]
        buf = (ctypes.c_int * max(total - start, 1))()
        n = checked(lib().cellm_sched_tokens(self._h, int(request_id), int(start), buf, len(buf)), SchedulerError)
        out = list(buf[:n])
        return out if count is None else out[:count]

    def stats(self) -> dict:
        buf = (ctypes.c_longlong * 6)()
        lib().cellm_sched_stats(self._h, buf)
        return {"waiting": buf[0], "running": buf[1], "steps": buf[2], "tokens": buf[3],
                "preemptions": buf[4], "idle": bool(buf[5])}
