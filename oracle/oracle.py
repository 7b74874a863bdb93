"""ctypes front end of the CPU oracle (test infrastructure; never imported by the package).

Mirrors the operator names of the reference's provider (``hash_join_v2``, ``dedup``,
``union_many_gpu``, ``diff_gpu``, ``sort``) and its executor (``register_relation``,
``put_relation``, ``execute_plan``, ``get``) so tests can run the same scenario on both sides.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libxlog_oracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "xlog_oracle.cpp")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        L = _lib
        P = C.c_void_p
        L.xo_rel_from_cols.restype = P
        L.xo_rel_from_cols.argtypes = [C.c_uint32, C.c_uint32, C.POINTER(P), C.c_uint64]
        L.xo_rel_rows.restype = C.c_uint64
        L.xo_rel_rows.argtypes = [P]
        L.xo_rel_arity.restype = C.c_uint32
        L.xo_rel_arity.argtypes = [P]
        L.xo_rel_width.restype = C.c_uint32
        L.xo_rel_width.argtypes = [P]
        L.xo_rel_canonical.argtypes = [P]
        L.xo_rel_to_cols.argtypes = [P, C.POINTER(P)]
        L.xo_rel_free.argtypes = [P]
        U = C.POINTER(C.c_uint32)
        for name, args in (("xo_sort", [P, U, C.c_uint32]), ("xo_dedup", [P, U, C.c_uint32]),
                           ("xo_union", [C.POINTER(P), C.c_uint32]), ("xo_diff", [P, P]),
                           ("xo_hash_join", [P, P, U, U, C.c_uint32, C.c_int])):
            getattr(L, name).restype = P
            getattr(L, name).argtypes = args
        L.xo_exec_new.restype = P
        L.xo_exec_new.argtypes = [C.c_uint64]
        L.xo_exec_free.argtypes = [P]
        L.xo_register.argtypes = [P, C.c_uint32, C.c_char_p]
        L.xo_put.argtypes = [P, C.c_char_p, P]
        L.xo_get.restype = P
        L.xo_get.argtypes = [P, C.c_char_p]
        L.xo_error.restype = C.c_char_p
        L.xo_error.argtypes = [P]
        L.xo_iterations.restype = C.c_uint64
        L.xo_iterations.argtypes = [P]
        L.xo_candidates.restype = C.c_uint64
        L.xo_candidates.argtypes = [P]
        L.xo_execute_plan.argtypes = [P, C.c_void_p]
    return _lib


def set_threads(n: int) -> None:
    lib().xo_set_threads(int(n))


def _u32s(xs):
    return (C.c_uint32 * max(len(xs), 1))(*xs)


def _to_ordered(c: np.ndarray) -> np.ndarray:
    """Order-preserving unsigned image of a typed column: sign flip for signed integers, IEEE
    totalOrder for floats (the reference's key transforms, kernels/sort.cu:296-448,
    kernels/totalorder.cuh); unsigned columns pass through."""
    k = c.dtype.kind
    if k == "u":
        return c
    u = c.view(np.uint32 if c.dtype.itemsize == 4 else np.uint64)
    sign = u.dtype.type(1) << u.dtype.type(c.dtype.itemsize * 8 - 1)
    if k == "i":
        return u ^ sign
    return np.where(u & sign, ~u, u | sign)


def _from_ordered(u: np.ndarray, dtype) -> np.ndarray:
    dtype = np.dtype(dtype)
    if dtype.kind == "u":
        return u
    sign = u.dtype.type(1) << u.dtype.type(dtype.itemsize * 8 - 1)
    raw = (u ^ sign) if dtype.kind == "i" else np.where(u & sign, u ^ sign, ~u)
    return raw.astype(u.dtype).view(dtype)


class OracleRel:
    """Host relation: equal-length numpy columns, held in one width class (4 or 8 bytes; mixed
    widths are widened to 8).  Signed and floating columns are held as their order-preserving
    unsigned images."""

    def __init__(self, handle, dtypes=None):
        if not handle:
            raise ValueError("oracle operator rejected its inputs")
        self._h = handle
        self.dtypes = dtypes

    @classmethod
    def from_columns(cls, cols, dtype=None, arity=None):
        if dtype is not None:
            cols = [np.ascontiguousarray(c, dtype=dtype) for c in cols]
        else:
            cols = [np.ascontiguousarray(c) for c in cols]
            cols = [c if c.dtype.itemsize in (4, 8) and c.dtype.kind in "uif" else c.astype(np.uint32) for c in cols]
        dtypes = [c.dtype for c in cols]
        width = dtypes[0].itemsize if dtypes else (np.dtype(dtype).itemsize if dtype is not None else 4)
        ucols = [np.ascontiguousarray(_to_ordered(c)) for c in cols]
        if any(d.itemsize != width for d in dtypes):
            # 4- and 8-byte columns together: the unsigned images of the narrow ones are widened
            # (same order, same equality); `columns` narrows them again
            width = 8
            ucols = [np.ascontiguousarray(u.astype(np.uint64)) for u in ucols]
        arity = len(cols) if arity is None else arity
        rows = len(cols[0]) if cols else 0
        ptrs = (C.c_void_p * max(arity, 1))(*[c.ctypes.data for c in ucols])
        return cls(lib().xo_rel_from_cols(arity, width, ptrs, rows), dtypes)

    def _like(self, handle, dtypes=None):
        return OracleRel(handle, self.dtypes if dtypes is None else dtypes)

    @property
    def rows(self):
        return lib().xo_rel_rows(self._h)

    @property
    def arity(self):
        return lib().xo_rel_arity(self._h)

    @property
    def canonical(self):
        return bool(lib().xo_rel_canonical(self._h))

    def columns(self):
        dt = np.uint32 if lib().xo_rel_width(self._h) == 4 else np.uint64
        cols = [np.empty(self.rows, dtype=dt) for _ in range(self.arity)]
        ptrs = (C.c_void_p * max(self.arity, 1))(*[c.ctypes.data for c in cols])
        lib().xo_rel_to_cols(self._h, ptrs)
        if self.dtypes and len(self.dtypes) == len(cols):
            cols = [_from_ordered(c.astype(np.uint32) if np.dtype(d).itemsize == 4 and c.dtype.itemsize == 8 else c, d)
                    for c, d in zip(cols, self.dtypes)]
        return cols

    def tuples(self):
        return list(zip(*[c.tolist() for c in self.columns()])) if self.arity else []

    def __del__(self):
        if getattr(self, "_h", None):
            lib().xo_rel_free(self._h)
            self._h = None


def _same_types(rels):
    d0 = [np.dtype(d) for d in (rels[0].dtypes or [])]
    for r in rels[1:]:
        if [np.dtype(d) for d in (r.dtypes or [])] != d0:
            raise ValueError("incompatible column types")


def sort(r, keys):
    return r._like(lib().xo_sort(r._h, _u32s(keys), len(keys)))


def dedup(r, keys=()):
    return r._like(lib().xo_dedup(r._h, _u32s(keys), len(keys)))


def union_many(rels):
    if not rels:
        raise ValueError("union of no inputs")
    _same_types(rels)
    arr = (C.c_void_p * max(len(rels), 1))(*[r._h for r in rels])
    return rels[0]._like(lib().xo_union(arr, len(rels)))


def diff(a, b):
    _same_types([a, b])
    return a._like(lib().xo_diff(a._h, b._h))


def groupby_columns(cols, key_cols, aggs):
    """groupby_multi_agg on host columns (crates/xlog-cuda/src/provider/groupby.rs:66-819): one row
    per distinct key, ascending by key; key columns, then per (value column, op) with op 0 count,
    1 sum, 2 min, 3 max: count and sum as u64, min and max in the width of the value column.
    Plain numpy: lexicographic sort of the key columns, boundaries, ``reduceat``."""
    cols = [np.asarray(c) for c in cols]
    n = len(cols[0]) if cols else 0
    out_types = [cols[k].dtype for k in key_cols] + [np.dtype(np.uint64) if op in (0, 1) else (np.dtype(np.uint64) if cols[v].dtype == np.uint64 else np.dtype(np.uint32)) for v, op in aggs]
    if n == 0:
        return [np.zeros(0, dtype=t) for t in out_types]
    order = np.lexsort([cols[k] for k in reversed(list(key_cols))])
    keys = [cols[k][order] for k in key_cols]
    head = np.ones(n, dtype=bool)
    head[1:] = np.zeros(n - 1, dtype=bool)
    for k in keys:
        head[1:] |= k[1:] != k[:-1]
    starts = np.flatnonzero(head)
    out = [k[starts] for k in keys]
    for (v, op), t in zip(aggs, out_types[len(key_cols):]):
        vals = cols[v][order].astype(np.uint64)
        if op == 0:
            r = np.diff(np.append(starts, n)).astype(np.uint64)
        elif op == 1:
            r = np.add.reduceat(vals, starts)          # wraps modulo 2^64 like the device sum
        elif op == 2:
            r = np.minimum.reduceat(vals, starts)
        else:
            r = np.maximum.reduceat(vals, starts)
        out.append(r.astype(t))
    return out


def hash_join(l, r, lk, rk, join_type=0):
    dt = (l.dtypes or []) + (r.dtypes or []) if join_type == 0 else l.dtypes
    return OracleRel(lib().xo_hash_join(l._h, r._h, _u32s(lk), _u32s(rk), len(lk), join_type), dt)


class OracleExecutor:
    """Executor::{register_relation, put_relation, execute_plan, store().get}
    (crates/xlog-runtime/src/executor/mod.rs:1242,587,1404,562) on the CPU."""

    def __init__(self, max_iterations: int = 0):
        self._h = lib().xo_exec_new(max_iterations)

    def register_relation(self, rel_id, name):
        lib().xo_register(self._h, rel_id, name.encode())

    def put_relation(self, name, rel):
        lib().xo_put(self._h, name.encode(), rel._h)

    def get(self, name):
        return OracleRel(lib().xo_get(self._h, name.encode()))

    def execute_plan(self, compiled_plan):
        st = lib().xo_execute_plan(self._h, C.addressof(compiled_plan.c))
        if st != 0:
            raise RuntimeError(f"oracle status {st}: {lib().xo_error(self._h).decode()}")

    @property
    def iterations(self):
        return lib().xo_iterations(self._h)

    @property
    def candidates(self):
        return lib().xo_candidates(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().xo_exec_free(self._h)
            self._h = None


def run_program(plan, inputs, outputs, max_iterations=0):
    """Evaluate ``plan`` on ``inputs`` (name -> list of numpy columns); returns
    (dict name -> list of columns, executor)."""
    ex = OracleExecutor(max_iterations)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    for name, cols in inputs.items():
        ex.put_relation(name, OracleRel.from_columns(cols))
    cp = plan.compile()
    ex.execute_plan(cp)
    # typed columns are held as order-preserving unsigned images: decode the outputs with the column
    # types the plan declares for its heads (inputs keep the types they came with)
    np_of = {0: np.uint32, 1: np.uint64, 2: np.int32, 3: np.int64, 4: np.float32, 5: np.float64, 7: np.uint32}
    types = {name: [np.asarray(c).dtype for c in cols] for name, cols in inputs.items()}
    for s in plan.sccs:
        for r in s.rules:
            types.setdefault(r.head, [np.dtype(np_of[t]) for t in r.head_types])
    out = {}
    for o in outputs:
        rel = ex.get(o)
        if o in types and len(types[o]) == rel.arity:
            rel.dtypes = types[o]
        out[o] = rel.columns()
    return out, ex
