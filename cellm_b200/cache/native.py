"""ctypes binding to the host runtime (allocator, cache manager, scheduler)."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p

from ..csrc import build as _build

_lib = None


class CacheError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        l = _build.load("runtime")
        IP, LP = POINTER(c_int), POINTER(c_longlong)
        sig = {
            "cellm_last_error": ([], c_char_p),
            "cellm_cache_create": ([c_int, c_int, IP, IP, c_int], c_void_p),
            "cellm_cache_destroy": ([c_void_p], None),
            "cellm_cache_add": ([c_void_p, c_longlong], c_int),
            "cellm_cache_reserve": ([c_void_p, c_longlong, c_int], c_int),
            "cellm_cache_can_reserve": ([c_void_p, c_longlong, c_int], c_int),
            "cellm_cache_commit": ([c_void_p, c_longlong, c_int], c_int),
            "cellm_cache_release": ([c_void_p, c_longlong], c_int),
            "cellm_cache_has": ([c_void_p, c_longlong], c_int),
            "cellm_cache_tokens": ([c_void_p, c_longlong], c_int),
            "cellm_cache_slot": ([c_void_p, c_longlong], c_int),
            "cellm_cache_block_table": ([c_void_p, c_longlong, c_int, c_void_p, c_int], c_int),
            "cellm_cache_free_pages": ([c_void_p, c_int], c_int),
            "cellm_cache_free_slots": ([c_void_p], c_int),
            "cellm_cache_live": ([c_void_p], c_int),
            "cellm_cache_pages_for": ([c_void_p, c_int, c_int, c_int], c_int),
            "cellm_alloc_create": ([c_int], c_void_p),
            "cellm_alloc_destroy": ([c_void_p], None),
            "cellm_alloc_alloc": ([c_void_p], c_int),
            "cellm_alloc_alloc_n": ([c_void_p, c_int, IP], c_int),
            "cellm_alloc_free": ([c_void_p, c_int], c_int),
            "cellm_alloc_free_count": ([c_void_p], c_int),
            "cellm_alloc_is_free": ([c_void_p, c_int], c_int),
            "cellm_sched_create": ([c_void_p, c_int, c_int, c_int], c_void_p),
            "cellm_sched_destroy": ([c_void_p], None),
            "cellm_sched_add": ([c_void_p, c_longlong, IP, c_int, c_int], c_int),
            "cellm_sched_schedule": ([c_void_p], c_int),
            "cellm_sched_plan_entries": ([c_void_p, LP, IP, IP, IP, c_int], c_int),
            "cellm_sched_plan_preempted": ([c_void_p, LP, c_int], c_int),
            "cellm_sched_plan_admitted": ([c_void_p, LP, IP, c_int], c_int),
            "cellm_sched_step_done": ([c_void_p], c_int),
            "cellm_sched_plan_shape": ([c_void_p, IP], c_int),
            "cellm_sched_plan_fill": ([c_void_p, c_void_p, c_int, c_int, c_int], c_int),
            "cellm_sched_append_rows": ([c_void_p, c_void_p, c_void_p, c_void_p, c_int], c_int),
            "cellm_sched_append": ([c_void_p, c_longlong, c_int, c_int], c_int),
            "cellm_sched_resolve_rows": ([c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int], c_int),
            "cellm_sched_cancel": ([c_void_p, c_longlong], c_int),
            "cellm_sched_forget": ([c_void_p, c_longlong], c_int),
            "cellm_sched_has": ([c_void_p, c_longlong], c_int),
            "cellm_sched_info": ([c_void_p, c_longlong, IP], c_int),
            "cellm_sched_tokens": ([c_void_p, c_longlong, c_int, IP, c_int], c_int),
            "cellm_sched_finish_reason": ([c_void_p, c_longlong], c_char_p),
            "cellm_sched_stats": ([c_void_p, LP], None),
        }
        for name, (args, res) in sig.items():
            f = getattr(l, name)
            f.argtypes, f.restype = args, res
        _lib = l
    return _lib


def last_error() -> str:
    return lib().cellm_last_error().decode()


def checked(code: int, exc=CacheError) -> int:
    if code < 0:
        raise exc(last_error())
    return code


def int_array(values):
    return (ctypes.c_int * len(values))(*values)
