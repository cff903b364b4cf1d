"""Python face of the host runtime (``csrc/host/*.cpp``): page pools, cache bookkeeping, step
packing and the scheduler's decisions are C++ behind a C interface, built at first use by
``csrc/build.py`` and called through ctypes.  No GPU is involved; everything here runs on a
machine without one."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int32, c_longlong, c_void_p

from .csrc.build import host_library_path

# Status codes of csrc/host/page_pool.hpp
OK = 0
OUT_OF_PAGES, NOT_OF_POOL, FREED_TWICE, ALREADY_LIVE, OUT_OF_SLOTS = -1, -2, -3, -4, -5
UNKNOWN_REQUEST, TOO_LONG, EXCEEDS_RESERVED, NO_PAGE, BAD_ARGUMENT, BOOKS_WRONG = -6, -7, -8, -9, -10, -11

_INT_P = POINTER(c_int)
_I32_P = POINTER(c_int32)
_I64_P = POINTER(c_longlong)

_SIGNATURES = {
    "egh_pool_create": (c_void_p, [c_int]),
    "egh_pool_destroy": (None, [c_void_p]),
    "egh_pool_alloc": (c_int, [c_void_p, c_int, c_void_p]),
    "egh_pool_free": (c_int, [c_void_p, c_void_p, c_int, _INT_P]),
    "egh_pool_check": (c_int, [c_void_p]),
    "egh_pool_stat": (c_longlong, [c_void_p, c_int]),
    "egh_cache_create": (c_void_p, [c_int, c_int, c_int]),
    "egh_cache_destroy": (None, [c_void_p]),
    "egh_cache_add_group": (c_int, [c_void_p, c_int, c_int]),
    "egh_cache_group_pool": (c_void_p, [c_void_p, c_int]),
    "egh_cache_group_table": (_I32_P, [c_void_p, c_int]),
    "egh_cache_begin": (c_int, [c_void_p, c_longlong]),
    "egh_cache_end": (c_int, [c_void_p, c_longlong]),
    "egh_cache_take_fresh": (c_int, [c_void_p, c_void_p, c_int]),
    "egh_cache_query": (c_longlong, [c_void_p, c_longlong, c_int]),
    "egh_cache_max_length": (c_longlong, [c_void_p, c_int, c_void_p]),
    "egh_cache_pages_needed": (c_int, [c_void_p, c_longlong, c_longlong, c_void_p]),
    "egh_cache_can_reserve": (c_int, [c_void_p, c_longlong, c_longlong, c_int]),
    "egh_cache_reserve": (c_int, [c_void_p, c_longlong, c_longlong, c_void_p]),
    "egh_cache_commit": (c_int, [c_void_p, c_longlong, c_longlong]),
    "egh_cache_free_slots": (c_int, [c_void_p]),
    "egh_cache_slot_positions": (c_int, [c_void_p, c_int, c_longlong, c_longlong, c_int, c_void_p]),
    "egh_cache_live": (c_int, [c_void_p, c_void_p, c_int]),
    "egh_cache_check": (c_int, [c_void_p, c_char_p, c_int]),
    "egh_step_reserve": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "egh_step_bound": (c_longlong, [c_void_p, c_int, c_longlong, c_longlong, c_int]),
    "egh_step_pack": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                              c_void_p, c_longlong, c_void_p, c_void_p, c_void_p]),
    "egh_replay_pack": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_longlong,
                                c_void_p, c_void_p, c_int]),
    "egh_sched_create": (c_void_p, [c_void_p, c_longlong, c_longlong, c_int, c_int, c_longlong, c_longlong]),
    "egh_sched_destroy": (None, [c_void_p]),
    "egh_sched_add": (c_longlong, [c_void_p, c_longlong, c_longlong]),
    "egh_sched_has_work": (c_int, [c_void_p]),
    "egh_sched_schedule": (c_int, [c_void_p, c_void_p, c_int]),
    "egh_sched_launched": (c_int, [c_void_p, c_void_p, c_int]),
    "egh_sched_resolve": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "egh_sched_advance": (c_int, [c_void_p, c_longlong, c_longlong]),
    "egh_sched_request": (c_int, [c_void_p, c_longlong, c_void_p]),
    "egh_sched_list": (c_int, [c_void_p, c_int, c_void_p, c_int]),
    "egh_sched_stats": (None, [c_void_p, c_void_p]),
    "egh_sched_forget": (None, [c_void_p, c_longlong]),
    "egh_bpe_create": (c_void_p, []),
    "egh_bpe_destroy": (None, [c_void_p]),
    "egh_bpe_add_tokens": (None, [c_void_p, c_char_p, c_void_p, c_void_p, c_int]),
    "egh_bpe_add_merges": (None, [c_void_p, c_char_p, c_void_p, c_char_p, c_void_p, c_int]),
    "egh_bpe_add_specials": (None, [c_void_p, c_char_p, c_void_p, c_int]),
    "egh_bpe_set_bos": (None, [c_void_p, c_int]),
    "egh_bpe_encode": (c_longlong, [c_void_p, c_char_p, c_longlong, c_void_p, c_longlong]),
    "egh_bpe_tokenize": (c_longlong, [c_void_p, c_char_p, c_longlong, c_void_p, c_longlong]),
    "egh_bpe_decode": (c_longlong, [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong]),
}

_lib = None


class HostRuntimeError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = host_library_path()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise HostRuntimeError(f"cannot load the host runtime {path}: {e}") from None
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib
