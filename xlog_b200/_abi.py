"""ctypes mirror of include/xlb.h (types only; no library is loaded here)."""
from __future__ import annotations

import ctypes as C

XLB_MAX_ARITY = 8
XLB_MAX_KEYS = 2
XLB_UNIQUE_ID_BYTES = 128

# xlb_status
OK, ERR_INVALID, ERR_TYPE, ERR_RESOURCE_EXHAUSTED, ERR_CAPACITY, ERR_ITER_LIMIT, ERR_CUDA, \
    ERR_NCCL, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_NOT_FOUND = range(11)
STATUS_NAMES = ["OK", "INVALID", "TYPE", "RESOURCE_EXHAUSTED", "CAPACITY", "ITER_LIMIT", "CUDA",
                "NCCL", "TIMEOUT", "UNSUPPORTED", "NOT_FOUND"]

# xlb_type (crates/xlog-core/src/types.rs:33-62)
U32, U64, I32, I64, F32, F64, BOOL, SYMBOL = range(8)
# xlb_join_type
JOIN_INNER, JOIN_SEMI, JOIN_ANTI = range(3)
# xlb_agg_op (AggOp, crates/xlog-ir/src/rir.rs)
AGG_COUNT, AGG_SUM, AGG_MIN, AGG_MAX = range(4)
# xlb_node_kind
NODE_SCAN, NODE_FILTER, NODE_PROJECT, NODE_JOIN, NODE_UNION, NODE_DIFF, NODE_DISTINCT = 1, 2, 3, 4, 5, 6, 7
# xlb_cmp
EQ, NE, LT, LE, GT, GE = range(6)

FLAG_PROFILE = 1
FLAG_NO_DENSE = 2
FLAG_KEEP_DELTAS = 4
FLAG_SHUFFLE_ONLY = 8
FLAG_NO_TUPLE_SET = 16
FLAG_GENERAL_ONLY = 32


class Schema(C.Structure):
    _fields_ = [("arity", C.c_uint32), ("types", C.c_uint8 * XLB_MAX_ARITY)]

    @classmethod
    def of(cls, types):
        s = cls()
        s.arity = len(types)
        for i, t in enumerate(types):
            s.types[i] = t
        return s


class Config(C.Structure):
    _fields_ = [("device", C.c_int32), ("memory_budget_bytes", C.c_uint64),
                ("max_iterations", C.c_uint64), ("join_chunk_tuples", C.c_uint64),
                ("flags", C.c_uint32)]


class Node(C.Structure):
    pass


Node._fields_ = [
    ("kind", C.c_uint32), ("rel_id", C.c_uint32),
    ("input", C.POINTER(Node)), ("left", C.POINTER(Node)), ("right", C.POINTER(Node)),
    ("n_keys", C.c_uint32),
    ("left_keys", C.c_uint32 * XLB_MAX_KEYS), ("right_keys", C.c_uint32 * XLB_MAX_KEYS),
    ("n_cols", C.c_uint32), ("cols", C.c_uint32 * XLB_MAX_ARITY),
    ("cmp", C.c_uint32), ("cmp_lhs_col", C.c_uint32), ("cmp_rhs_is_const", C.c_uint32),
    ("cmp_rhs", C.c_uint64),
    ("inputs", C.POINTER(C.POINTER(Node))), ("n_inputs", C.c_uint32), ("join_type", C.c_uint32),
]


class Rule(C.Structure):
    _fields_ = [("head", C.c_char_p), ("body", C.POINTER(Node)), ("head_schema", Schema)]


class Scc(C.Structure):
    _fields_ = [("id", C.c_uint32), ("is_recursive", C.c_uint32),
                ("rules", C.POINTER(Rule)), ("n_rules", C.c_uint32)]


class Plan(C.Structure):
    _fields_ = [("sccs", C.POINTER(Scc)), ("n_sccs", C.c_uint32)]


class RunStats(C.Structure):
    _fields_ = [("iterations", C.c_uint64), ("derived_tuples", C.c_uint64),
                ("candidate_tuples", C.c_uint64), ("kernel_launches", C.c_uint64),
                ("peak_bytes", C.c_uint64), ("ms_total", C.c_double), ("ms_join", C.c_double),
                ("ms_sort", C.c_double), ("ms_setops", C.c_double), ("ms_exchange", C.c_double),
                ("exchange_bytes", C.c_uint64), ("host_syncs", C.c_uint64),
                ("ms_host_wait", C.c_double), ("ms_host_total", C.c_double), ("ms_host_alloc", C.c_double)]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


class KernelProfile(C.Structure):
    _fields_ = [("name", C.c_char * 32), ("launches", C.c_uint64), ("bytes", C.c_uint64), ("ms", C.c_double)]
