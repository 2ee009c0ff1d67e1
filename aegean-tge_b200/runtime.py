"""ctypes binding of the host runtime (csrc/runtime.cpp): page pools, cache bookkeeping, scheduler and
step packing live in C++; the Python classes of the cache manager and the scheduler are views of
these objects.  The library is compiled in-tree at first use and needs no GPU.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int64, c_longlong, c_void_p
from typing import Optional

OK, EXHAUSTED, PAGE_ERROR, VALUE_ERROR, STUCK = 0, -1, -2, -3, -4


class PoolExhausted(RuntimeError):
    """No free page or state slot is left."""


class PageError(RuntimeError):
    """A page, slot or request was used in a way its state does not allow."""


class StepLayout(ctypes.Structure):
    _fields_ = [(name, c_int) for name in
                ("num_tokens", "num_seqs", "num_rows", "max_q_len", "max_ctx_len", "total_ints",
                 "token_ids", "positions", "seq_of_token", "q_start", "start_pos", "ctx_len", "slots", "logit_rows")]
    _fields_ += [("table", c_int * 8), ("width", c_int * 8)]


_lib: Optional[ctypes.CDLL] = None
_INT_P = POINTER(c_int)
_I64_P = POINTER(c_int64)

_SIGNATURES = {
    "tge_rt_last_error": (c_char_p, []),
    "tge_rt_pool_create": (c_void_p, [c_int]),
    "tge_rt_pool_destroy": (None, [c_void_p]),
    "tge_rt_pool_capacity": (c_int, [c_void_p]),
    "tge_rt_pool_free_count": (c_int, [c_void_p]),
    "tge_rt_pool_allocate": (c_int, [c_void_p]),
    "tge_rt_pool_share": (c_int, [c_void_p, c_int]),
    "tge_rt_pool_release": (c_int, [c_void_p, c_int]),
    "tge_rt_pool_refcount": (c_int, [c_void_p, c_int]),
    "tge_rt_pool_check": (c_int, [c_void_p]),
    "tge_rt_cache_create": (c_void_p, [c_int, c_int]),
    "tge_rt_cache_destroy": (None, [c_void_p]),
    "tge_rt_cache_add_group": (c_int, [c_void_p, c_int]),
    "tge_rt_cache_set_pool_size": (c_int, [c_void_p, c_int, c_int]),
    "tge_rt_cache_pool": (c_void_p, [c_void_p, c_int]),
    "tge_rt_cache_groups": (c_int, [c_void_p]),
    "tge_rt_cache_free_slots": (c_int, [c_void_p]),
    "tge_rt_cache_live_count": (c_int, [c_void_p]),
    "tge_rt_cache_live_requests": (c_int, [c_void_p, _I64_P, c_int]),
    "tge_rt_cache_is_live": (c_int, [c_void_p, c_int64]),
    "tge_rt_cache_slot_of": (c_int, [c_void_p, c_int64]),
    "tge_rt_cache_tokens_of": (c_int, [c_void_p, c_int64]),
    "tge_rt_cache_computed": (c_int, [c_void_p, c_int64]),
    "tge_rt_cache_admit": (c_int, [c_void_p, c_int64]),
    "tge_rt_cache_can_grow": (c_int, [c_void_p, c_int64, c_int]),
    "tge_rt_cache_fits_empty_pool": (c_int, [c_void_p, c_int]),
    "tge_rt_cache_pages_missing": (c_int, [c_void_p, c_int64, c_int, _INT_P]),
    "tge_rt_cache_grow": (c_int, [c_void_p, c_int64, c_int]),
    "tge_rt_cache_set_computed": (c_int, [c_void_p, c_int64, c_int]),
    "tge_rt_cache_release_behind_window": (c_int, [c_void_p, c_int64, c_int]),
    "tge_rt_cache_free": (c_int, [c_void_p, c_int64]),
    "tge_rt_cache_table_length": (c_int, [c_void_p, c_int, c_int64]),
    "tge_rt_cache_table": (c_int, [c_void_p, c_int, c_int64, _INT_P, c_int]),
    "tge_rt_cache_fill_block_table": (c_int, [c_void_p, c_int, _I64_P, c_int, c_void_p, c_int]),
    "tge_rt_cache_check": (c_int, [c_void_p]),
    "tge_rt_cache_max_context": (c_int, [c_void_p, _I64_P, _INT_P, c_int]),
    "tge_rt_cache_advance": (c_int, [c_void_p, _I64_P, _INT_P, c_int]),
    "tge_rt_step_pack": (c_int, [c_void_p, c_int, _I64_P, POINTER(c_void_p), _INT_P, POINTER(c_void_p), _INT_P, c_int,
                                 c_int, c_int, c_int, c_void_p, c_longlong, POINTER(StepLayout)]),
    "tge_rt_sched_create": (c_void_p, [c_void_p, c_int, c_int, c_int, c_int, _INT_P, c_int]),
    "tge_rt_sched_destroy": (None, [c_void_p]),
    "tge_rt_sched_add": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int]),
    "tge_rt_sched_has_work": (c_int, [c_void_p]),
    "tge_rt_sched_waiting": (c_int, [c_void_p, _I64_P, c_int]),
    "tge_rt_sched_running": (c_int, [c_void_p, _I64_P, c_int]),
    "tge_rt_sched_schedule": (c_int, [c_void_p]),
    "tge_rt_sched_plan": (c_int, [c_void_p, _I64_P, _INT_P, _INT_P, _INT_P, c_int]),
    "tge_rt_sched_plan_preempted": (c_int, [c_void_p, _I64_P, c_int]),
    "tge_rt_sched_pack": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_longlong, POINTER(StepLayout)]),
    "tge_rt_sched_update": (c_int, [c_void_p, c_void_p, c_int, _I64_P, _INT_P, c_int]),
    "tge_rt_sched_request_info": (c_int, [c_void_p, c_int64, _INT_P, _INT_P, _INT_P, _INT_P]),
    "tge_rt_sched_tokens": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p]),
    "tge_rt_sched_forget": (c_int, [c_void_p, c_int64]),
    "tge_rt_sched_counter": (c_longlong, [c_void_p, c_int]),
    "tge_rt_random_fill": (c_int, [c_void_p, c_int, c_longlong, c_longlong, ctypes.c_ulonglong, c_int, ctypes.c_float,
                                   c_int, ctypes.c_uint, c_int]),
}


def lib() -> ctypes.CDLL:
    """The runtime library, built and loaded at first use."""
    global _lib
    if _lib is None:
        from .csrc.build import build_runtime
        handle = ctypes.CDLL(build_runtime())
        for name, (restype, argtypes) in _SIGNATURES.items():
            function = getattr(handle, name)
            function.restype = restype
            function.argtypes = argtypes
        _lib = handle
    return _lib


def library_path() -> Optional[str]:
    return None if _lib is None else _lib._name


def check(code: int) -> int:
    """Turns a negative return code into the matching exception; passes counts through."""
    if code >= 0:
        return code
    message = lib().tge_rt_last_error().decode("utf-8", "replace")
    if code == EXHAUSTED:
        raise PoolExhausted(message)
    if code == PAGE_ERROR:
        raise PageError(message)
    if code == VALUE_ERROR:
        raise ValueError(message)
    raise RuntimeError(message)
