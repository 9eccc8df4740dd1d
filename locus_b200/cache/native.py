"""The host library (``csrc/host_core.cpp``: pools, page tables, step assembly, scheduler) loaded with
ctypes, its entry points declared.  Compiled on first use like the kernel modules; there is
no Python stand-in: without a C++ compiler the import of the cache fails with the build error."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_int64, c_void_p

from ..csrc import build

_lib = None

P_INT = POINTER(c_int)
P_I64 = POINTER(c_int64)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = build.load("host_core")
        sig = {
            "locus_pool_new": (c_void_p, [c_int]),
            "locus_pool_delete": (None, [c_void_p]),
            "locus_pool_total": (c_int, [c_void_p]),
            "locus_pool_free": (c_int, [c_void_p]),
            "locus_pool_refs": (c_int, [c_void_p, c_int]),
            "locus_pool_allocate": (c_int, [c_void_p]),
            "locus_pool_release": (c_int, [c_void_p, c_int]),
            "locus_pool_retain": (c_int, [c_void_p, c_int]),
            "locus_cache_new": (c_void_p, [c_int, P_INT, c_int, P_INT, c_int, c_int]),
            "locus_cache_total_pages": (c_int, [c_void_p, c_int]),
            "locus_cache_pages_needed": (c_int, [c_void_p, c_int, c_int, c_int]),
            "locus_cache_delete": (None, [c_void_p]),
            "locus_cache_table_width": (c_int, [c_void_p]),
            "locus_cache_free_pages": (c_int, [c_void_p, c_int]),
            "locus_cache_page_refs": (c_int, [c_void_p, c_int, c_int]),
            "locus_cache_slots_free": (c_int, [c_void_p]),
            "locus_cache_slots_total": (c_int, [c_void_p]),
            "locus_cache_open": (c_int64, [c_void_p]),
            "locus_cache_is_open": (c_int, [c_void_p, c_int64]),
            "locus_cache_n_tokens": (c_int, [c_void_p, c_int64]),
            "locus_cache_state_slot": (c_int, [c_void_p, c_int64]),
            "locus_cache_capacity": (c_int, [c_void_p, c_int64]),
            "locus_cache_table": (c_int, [c_void_p, c_int64, c_int, P_INT, c_int]),
            "locus_cache_ensure": (c_int, [c_void_p, c_int64, c_int]),
            "locus_cache_commit": (c_int, [c_void_p, c_int64, c_int, P_INT, c_int]),
            "locus_cache_release": (c_int, [c_void_p, c_int64, P_INT, c_int]),
            "locus_cache_check": (c_int, [c_void_p, P_INT]),
            "locus_step_build": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
            "locus_plan_query_tiles": (c_int, [c_int, c_void_p, c_int, c_int, c_void_p, c_int64]),
            "locus_sort_tiles_by_position": (None, [c_int, c_void_p, c_void_p]),
            "locus_plan_segments_with": (c_int, [c_int, c_void_p, c_int, c_void_p, c_int64]),
        }
        sig.update({
            "locus_sched_new": (c_void_p, [c_void_p, c_int, c_int, c_int, c_int, c_int]),
            "locus_sched_delete": (None, [c_void_p]),
            "locus_sched_add": (c_int, [c_void_p, c_int64, c_int]),
            "locus_sched_forget": (None, [c_void_p, c_int64]),
            "locus_sched_admit": (c_int, [c_void_p]),
            "locus_sched_plan": (c_int, [c_void_p, P_I64, c_int]),
            "locus_sched_fed": (None, [c_void_p, c_int64, c_int]),
            "locus_sched_token": (None, [c_void_p, c_int64, c_int]),
            "locus_sched_events": (c_int, [c_void_p, P_I64, c_int]),
            "locus_sched_freed": (c_int, [c_void_p, P_INT, c_int]),
            "locus_sched_queue": (c_int, [c_void_p, c_int, P_I64, c_int]),
            "locus_sched_count": (c_int, [c_void_p, c_int]),
        })
        for name, (res, args) in sig.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib
