"""Host-side mirror of the reference's kernel provider, over the C ABI.

Method names, argument meaning and error behaviour follow ``CudaKernelProvider``
(crates/xlog-cuda/src/provider/relational.rs): ``hash_join_v2`` (:2926), ``dedup`` (:238),
``union_gpu`` / ``union_many_gpu`` (:822, :859), ``diff_gpu`` (:1102), ``sort`` (:1881),
``clone_buffer`` (:6113), plus ``create_buffer_from_slices`` (provider/io.rs:75),
``device_row_count`` (provider/mod.rs:2823) and ``download_column`` (provider/transfer.rs:22).
Every call goes through libxlb.so; nothing is computed on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _abi as A
from .lib import XlbError, load

_NP = {A.U32: np.uint32, A.SYMBOL: np.uint32, A.U64: np.uint64, A.I32: np.int32, A.I64: np.int64,
       A.F32: np.float32, A.F64: np.float64, A.BOOL: np.uint8}
_CODE = {np.dtype(np.uint32): A.U32, np.dtype(np.uint64): A.U64, np.dtype(np.int32): A.I32, np.dtype(np.int64): A.I64,
         np.dtype(np.float32): A.F32, np.dtype(np.float64): A.F64, np.dtype(np.bool_): A.BOOL}


def _u32s(xs):
    return (C.c_uint32 * max(len(xs), 1))(*xs)


class Buffer:
    """Device relation handle (the reference's ``CudaBuffer``).  Owned unless borrowed."""

    def __init__(self, provider: "KernelProvider", handle, owned: bool = True):
        self.provider = provider
        self._h = C.c_void_p(handle) if not isinstance(handle, C.c_void_p) else handle
        self._owned = owned

    def num_rows(self) -> int:
        n = C.c_uint64()
        self.provider._check(self.provider._lib.xlb_rel_rows(self._h, C.byref(n)))
        return n.value

    def schema(self) -> list[int]:
        s = A.Schema()
        self.provider._check(self.provider._lib.xlb_rel_schema(self._h, C.byref(s)))
        return [s.types[i] for i in range(s.arity)]

    def arity(self) -> int:
        return len(self.schema())

    def is_canonical(self) -> bool:
        f = C.c_int()
        self.provider._check(self.provider._lib.xlb_rel_is_canonical(self._h, C.byref(f)))
        return bool(f.value)

    def release(self):
        """Give up ownership (the store took it)."""
        self._owned = False

    def free(self):
        if self._owned and self._h:
            self.provider._lib.xlb_rel_free(self._h)
        self._h = None

    def __del__(self):
        try:
            if self.provider._ctx:
                self.free()
        except Exception:
            pass


class KernelProvider:
    """One context on one GPU (``CudaKernelProvider::with_runtime``)."""

    def __init__(self, device: int = -1, memory_budget_bytes: int = 0, max_iterations: int = 0,
                 join_chunk_tuples: int = 0, profile: bool = False, flags: int = 0):
        self._lib = load()
        cfg = A.Config(device, memory_budget_bytes, max_iterations, join_chunk_tuples,
                       flags | (A.FLAG_PROFILE if profile else 0))
        ctx = C.c_void_p()
        st = self._lib.xlb_ctx_create(C.byref(cfg), C.byref(ctx))
        if st != A.OK:
            raise XlbError(st, self._lib.xlb_last_error(None).decode())
        self._ctx = ctx

    def close(self):
        if self._ctx:
            self._lib.xlb_ctx_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st: int):
        if st != A.OK:
            raise XlbError(st, self._lib.xlb_last_error(self._ctx).decode())

    def _out(self, fn, *args) -> Buffer:
        h = C.c_void_p()
        self._check(fn(self._ctx, *args, C.byref(h)))
        return Buffer(self, h)

    # ---- lifecycle / transfer ---------------------------------------------------------------
    def create_buffer_from_slices(self, cols: Sequence[np.ndarray], schema: Sequence[int] | None = None) -> Buffer:
        if schema is None:
            schema = [_CODE.get(np.asarray(c).dtype, A.U32) for c in cols]
        cols = [np.ascontiguousarray(c, dtype=_NP[t]) for c, t in zip(cols, schema)]
        rows = len(cols[0]) if cols else 0
        for c in cols:
            if len(c) != rows:
                raise ValueError("columns differ in length")
        s = A.Schema.of(list(schema))
        ptrs = (C.c_void_p * max(len(cols), 1))(*[c.ctypes.data for c in cols])
        return self._out(self._lib.xlb_rel_from_host, C.byref(s), ptrs, rows)

    create_buffer_from_u32_columns = create_buffer_from_slices

    def create_empty_buffer(self, schema: Sequence[int]) -> Buffer:
        s = A.Schema.of(list(schema))
        return self._out(self._lib.xlb_rel_empty, C.byref(s))

    def device_row_count(self, buf: Buffer) -> int:
        return buf.num_rows()

    def download(self, buf: Buffer) -> list[np.ndarray]:
        schema = buf.schema()
        n = buf.num_rows()
        cols = [np.empty(n, dtype=_NP[t]) for t in schema]
        ptrs = (C.c_void_p * max(len(cols), 1))(*[c.ctypes.data for c in cols])
        rows = C.c_uint64()
        self._check(self._lib.xlb_rel_to_host(self._ctx, buf._h, ptrs, n, C.byref(rows)))
        return cols

    def download_column(self, buf: Buffer, col: int) -> np.ndarray:
        return self.download(buf)[col]

    def checksum(self, buf: Buffer) -> tuple[int, int, int]:
        """(row count, XOR, low-32-bit sum) of the mixed rows, computed on the device: shards of a
        relation combine by adding the first and last and XOR-ing the middle (``xlb_rel_checksum``)."""
        d = (C.c_uint64 * 3)()
        self._check(self._lib.xlb_rel_checksum(self._ctx, buf._h, d))
        return int(d[0]), int(d[1]), int(d[2])

    def clone_buffer(self, buf: Buffer) -> Buffer:
        return self._out(self._lib.xlb_rel_clone, buf._h)

    # ---- operators --------------------------------------------------------------------------
    def hash_join_v2(self, left: Buffer, right: Buffer, left_keys, right_keys, join_type: int = A.JOIN_INNER) -> Buffer:
        if len(left_keys) != len(right_keys):
            raise XlbError(A.ERR_INVALID, "key lists differ in length")
        return self._out(self._lib.xlb_hash_join, left._h, right._h, _u32s(left_keys), _u32s(right_keys),
                         len(left_keys), join_type)

    def sort(self, buf: Buffer, key_cols) -> Buffer:
        return self._out(self._lib.xlb_sort, buf._h, _u32s(key_cols), len(key_cols))

    def dedup(self, buf: Buffer, key_cols=()) -> Buffer:
        return self._out(self._lib.xlb_dedup, buf._h, _u32s(key_cols), len(key_cols))

    def dedup_full_row(self, buf: Buffer) -> Buffer:
        return self.dedup(buf, ())

    def union_many_gpu(self, bufs: Sequence[Buffer]) -> Buffer:
        arr = (C.c_void_p * max(len(bufs), 1))(*[b._h for b in bufs])
        return self._out(self._lib.xlb_union, arr, len(bufs))

    def union_gpu(self, a: Buffer, b: Buffer) -> Buffer:
        return self.union_many_gpu([a, b])

    def diff_gpu(self, a: Buffer, b: Buffer) -> Buffer:
        return self._out(self._lib.xlb_diff, a._h, b._h)

    diff_full_row = diff_gpu

    def groupby_multi_agg(self, buf: Buffer, key_cols, aggs) -> Buffer:
        """``aggs``: (value column, A.AGG_*) pairs.  Key columns, then one column per aggregate;
        one row per group, ascending by key (provider/groupby.rs:66)."""
        aggs = list(aggs)
        return self._out(self._lib.xlb_groupby, buf._h, _u32s(key_cols), len(key_cols), _u32s([a[0] for a in aggs]),
                         _u32s([a[1] for a in aggs]), len(aggs))

    def groupby_agg(self, buf: Buffer, key_cols, agg: int, value_col: int) -> Buffer:
        return self.groupby_multi_agg(buf, key_cols, [(value_col, agg)])

    def memory_stats(self) -> tuple[int, int]:
        a, p = C.c_uint64(), C.c_uint64()
        self._check(self._lib.xlb_memory_stats(self._ctx, C.byref(a), C.byref(p)))
        return a.value, p.value

    def profile_enable(self, kernel: str | None) -> None:
        """Time every launch of ``kernel`` ("*" = all kernels, None = off) with CUDA events."""
        self._check(self._lib.xlb_profile_enable(self._ctx, kernel.encode() if kernel else None))

    def profile_read(self) -> dict:
        """name -> {launches, ms, bytes} since ``profile_enable``."""
        arr = (A.KernelProfile * 64)()
        n = C.c_uint32()
        self._check(self._lib.xlb_profile_read(self._ctx, arr, 64, C.byref(n)))
        return {arr[i].name.decode(): {"launches": arr[i].launches, "ms": arr[i].ms, "bytes": arr[i].bytes}
                for i in range(min(n.value, 64))}
