"""Loader for libxlb.so, the C ABI declared in include/xlb.h.

The CUDA path is the only path: if the shared library is missing, or no CUDA device is
present when a context is created, the caller gets an exception, never a host fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

from . import _abi as A

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("XLB_LIB") or os.path.join(_HERE, "libxlb.so")  # XLB_LIB: an alternative build, for A/B runs

P = C.c_void_p
U32P = C.POINTER(C.c_uint32)

# name -> (restype, argtypes): every symbol include/xlb.h declares
PROTOTYPES = {
    "xlb_ctx_create": (C.c_int, [C.POINTER(A.Config), C.POINTER(P)]),
    "xlb_ctx_destroy": (None, [P]),
    "xlb_last_error": (C.c_char_p, [P]),
    "xlb_memory_stats": (C.c_int, [P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "xlb_rel_from_host": (C.c_int, [P, C.POINTER(A.Schema), C.POINTER(P), C.c_uint64, C.POINTER(P)]),
    "xlb_rel_empty": (C.c_int, [P, C.POINTER(A.Schema), C.POINTER(P)]),
    "xlb_rel_rows": (C.c_int, [P, C.POINTER(C.c_uint64)]),
    "xlb_rel_schema": (C.c_int, [P, C.POINTER(A.Schema)]),
    "xlb_rel_is_canonical": (C.c_int, [P, C.POINTER(C.c_int)]),
    "xlb_rel_to_host": (C.c_int, [P, P, C.POINTER(P), C.c_uint64, C.POINTER(C.c_uint64)]),
    "xlb_rel_clone": (C.c_int, [P, P, C.POINTER(P)]),
    "xlb_rel_free": (None, [P]),
    "xlb_rel_checksum": (C.c_int, [P, P, C.POINTER(C.c_uint64)]),
    "xlb_hash_join": (C.c_int, [P, P, P, U32P, U32P, C.c_uint32, C.c_int, C.POINTER(P)]),
    "xlb_sort": (C.c_int, [P, P, U32P, C.c_uint32, C.POINTER(P)]),
    "xlb_dedup": (C.c_int, [P, P, U32P, C.c_uint32, C.POINTER(P)]),
    "xlb_union": (C.c_int, [P, C.POINTER(P), C.c_uint32, C.POINTER(P)]),
    "xlb_diff": (C.c_int, [P, P, P, C.POINTER(P)]),
    "xlb_groupby": (C.c_int, [P, P, C.POINTER(C.c_uint32), C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.c_uint32,
                              C.POINTER(P)]),
    "xlb_register_relation": (C.c_int, [P, C.c_uint32, C.c_char_p]),
    "xlb_store_put": (C.c_int, [P, C.c_char_p, P]),
    "xlb_store_get": (C.c_int, [P, C.c_char_p, C.POINTER(P)]),
    "xlb_store_remove": (C.c_int, [P, C.c_char_p]),
    "xlb_execute_plan": (C.c_int, [P, C.POINTER(A.Plan), C.POINTER(A.RunStats)]),
    "xlb_dedup_sorted_u64_static": (C.c_int, [P, C.c_uint64, P, P, P]),
    "xlb_dedup_sorted_u64_static_max": (C.c_uint64, []),
    "xlb_static_last_error": (C.c_char_p, []),
    "xlb_profile_enable": (C.c_int, [P, C.c_char_p]),
    "xlb_profile_read": (C.c_int, [P, C.POINTER(A.KernelProfile), C.c_uint32, C.POINTER(C.c_uint32)]),
    "xlb_comm_unique_id": (C.c_int, [C.POINTER(C.c_uint8)]),
    "xlb_comm_init": (C.c_int, [P, C.POINTER(C.c_uint8), C.c_uint32, C.c_uint32]),
    "xlb_owner_of": (C.c_uint32, [C.c_uint64, C.c_uint32]),
    "xlb_comm_mark_aborted_for_test": (C.c_int, [P]),
    "xlb_test_set_lookback": (C.c_int, [P, C.c_uint32, C.c_uint32]),
}


def build(verbose: bool = False) -> str:
    """Compile libxlb.so for sm_100a with nvcc (cross-compiles without a GPU)."""
    subprocess.check_call(["make", "-C", os.path.join(_HERE, "csrc"), "-j4"] + ([] if verbose else ["-s"]))
    return LIB_PATH


_lib = None


def load():
    """Load libxlb.so and bind every prototype.  Raises if the library was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                               "or `make -C xlog_b200/csrc` (there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class XlbError(RuntimeError):
    """A failing xlb_status, carrying the code and the library's message (XlogError)."""

    def __init__(self, status: int, message: str):
        name = A.STATUS_NAMES[status] if 0 <= status < len(A.STATUS_NAMES) else str(status)
        super().__init__(f"XLB_ERR_{name}: {message}")
        self.status = status
        self.message = message
