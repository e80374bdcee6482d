"""The host library (C++): page and slot pools, the cache manager's books, the
step builders and the scheduler.  Loaded with ctypes; built at first use by
`csrc/build.py` with the system's C++ compiler (no CUDA needed, so everything
here runs on a machine without a GPU).

Functions return a value >= 0 or a negative status; `check()` turns a negative
status into the Python exception its kind asks for, with the library's message.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int64, c_longlong, c_void_p

from .csrc import build as _build

ERR_ACCOUNTING, ERR_VALUE, ERR_OUT_OF_PAGES, ERR_REFUSED, ERR_UNKNOWN_REQUEST = -2, -3, -4, -5, -6

_LIB = None


class CacheAccountingError(RuntimeError):
    pass


class OutOfPages(RuntimeError):
    pass


class RequestRefused(ValueError):
    pass


def library() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        lib = ctypes.CDLL(_build.build_host())
        _declare(lib)
        _LIB = lib
    return _LIB


def last_error() -> str:
    return library().vxh_last_error().decode("utf-8", "replace")


def check(status: int) -> int:
    """`status` if it is not negative; else raises what the status stands for."""
    if status >= 0:
        return status
    msg = last_error()
    if status == ERR_ACCOUNTING:
        raise CacheAccountingError(msg)
    if status == ERR_OUT_OF_PAGES:
        raise OutOfPages(msg)
    if status == ERR_REFUSED:
        raise RequestRefused(msg)
    if status == ERR_UNKNOWN_REQUEST:
        raise KeyError(msg)
    raise ValueError(msg)


def _declare(lib: ctypes.CDLL) -> None:
    P, I, L = c_void_p, c_int, c_longlong
    PI, PI64 = POINTER(c_int), POINTER(c_int64)
    sig = {
        "vxh_last_error": (c_char_p, []),
        "vxh_pages_create": (P, [I]), "vxh_pages_destroy": (None, [P]), "vxh_pages_num_pages": (I, [P]),
        "vxh_pages_num_free": (I, [P]), "vxh_pages_alloc": (I, [P, I, PI]), "vxh_pages_incref": (I, [P, PI, I]),
        "vxh_pages_free": (I, [P, PI, I]), "vxh_pages_refcount": (I, [P, I]), "vxh_pages_free_list": (I, [P, PI, I]),
        "vxh_slots_create": (P, [I]), "vxh_slots_destroy": (None, [P]), "vxh_slots_num_slots": (I, [P]),
        "vxh_slots_num_free": (I, [P]), "vxh_slots_alloc": (I, [P]), "vxh_slots_free": (I, [P, I]),
        "vxh_cache_create": (P, [I, PI, I, I, I, I]), "vxh_cache_destroy": (None, [P]),
        "vxh_cache_pool": (P, [P, I]), "vxh_cache_slots": (P, [P]), "vxh_cache_add": (I, [P, c_int64]), "vxh_cache_has": (I, [P, c_int64]),
        "vxh_cache_num_requests": (L, [P]), "vxh_cache_request_ids": (L, [P, PI64, L]),
        "vxh_cache_length": (L, [P, c_int64]), "vxh_cache_max_length": (L, [P, I, PI64]), "vxh_cache_slot": (I, [P, c_int64]),
        "vxh_cache_table": (I, [P, c_int64, I, PI, I]), "vxh_cache_pages_needed": (I, [P, c_int64, L, PI]),
        "vxh_cache_can_reserve": (I, [P, c_int64, L]), "vxh_cache_reserve": (I, [P, c_int64, L]),
        "vxh_cache_commit": (I, [P, c_int64, L]), "vxh_cache_release": (I, [P, c_int64]),
        "vxh_cache_check": (I, [P]), "vxh_cache_reserve_many": (I, [P, I, PI64, PI]),
        "vxh_cache_commit_many": (I, [P, I, PI64, PI]),
        "vxh_build_step": (I, [P, I, PI64, PI, PI, PI, PI, I, I, c_void_p, PI64, PI64]),
        "vxh_fill_decode": (I, [P, I, I, PI64, PI, I, c_void_p, PI64, PI64]),
        "vxh_sched_create": (P, [P, I, L, L, L]), "vxh_sched_destroy": (None, [P]),
        "vxh_sched_max_model_len": (L, [P]), "vxh_sched_submit": (L, [P, PI, L, L, I, PI, I, PI, PI, I]),
        "vxh_sched_has_work": (I, [P]), "vxh_sched_plan": (I, [P, POINTER(c_longlong)]),
        "vxh_sched_plan_entries": (I, [P, PI64, PI64, PI64, PI, PI]), "vxh_sched_plan_ended": (I, [P, PI64]),
        "vxh_sched_plan_admitted": (I, [P, PI64, PI]),
        "vxh_sched_update": (I, [P, I, PI64, PI64, PI, PI, I, PI64, PI, PI]),
        "vxh_sched_finish": (I, [P, c_int64, I]), "vxh_sched_forget": (None, [P, c_int64]),
        "vxh_sched_cancel": (I, [P, c_int64]),
        "vxh_sched_list": (L, [P, I, PI64, L]), "vxh_sched_contains": (I, [P, I, c_int64]),
        "vxh_sched_request": (I, [P, c_int64, PI64]), "vxh_sched_request_tokens": (I, [P, c_int64, I, L, L, PI]),
        "vxh_sched_stats": (I, [P, PI64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args


def int_array(values) -> "ctypes.Array":
    values = list(values)
    return (c_int * len(values))(*values)


def int64_array(values) -> "ctypes.Array":
    values = list(values)
    return (c_int64 * len(values))(*values)
