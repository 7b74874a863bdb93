"""Rule shapes beyond the benchmark programs, CUDA path against the CPU oracle on random relations:
comparison filters (column/column and column/constant, all six operators), repeated variables,
unary relations as join partners, column swaps, constants that match nothing, empty inputs."""
import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200.executor import run_program
from xlog_b200.plan import CompiledRule, ExecutionPlan, Filter, Join, Project, Scan, Scc
from xlog_b200.provider import KernelProvider
from xlog_b200.workloads import splitmix64

pytestmark = pytest.mark.gpu
U1, U2 = (A.U32,), (A.U32, A.U32)


def _rel(n, cols, bits, seed):
    return [(splitmix64(seed + i, 0, n) >> np.uint64(64 - bits)).astype(np.uint32) for i in range(cols)]


def _plans():
    e, n, h = 0, 1, 2
    ids = {"e": e, "n": n, "h": h}

    def one(body, types, rec=False):
        return ExecutionPlan([Scc(0, rec, [CompiledRule("h", body, types)])], ids)

    shapes = {
        "self_loop": one(Project(Filter(Scan(e), A.EQ, 0, 1), [0]), U1),                       # h(X) :- e(X,X)
        "swap": one(Project(Scan(e), [1, 0]), U2),                                               # h(Y,X) :- e(X,Y)
        "unary_semi": one(Project(Join(Join(Scan(n), Scan(e), [0], [0]), Scan(n), [2], [0]), [0, 2]), U2),  # h(X,Y) :- n(X), e(X,Y), n(Y)
        "two_hop_ne": one(Project(Filter(Join(Scan(e), Scan(e), [1], [0]), A.NE, 0, 3), [0, 3]), U2),     # h(X,Z) :- e(X,Y), e(Y,Z), X != Z
        "const_none": one(Project(Filter(Scan(e), A.EQ, 0, 4_000_000_000, True), [1]), U1),     # no such constant
        "dup_head": one(Project(Scan(n), [0, 0]), U2),                                           # h(X,X) :- n(X)
    }
    for name, op in (("lt", A.LT), ("le", A.LE), ("gt", A.GT), ("ge", A.GE), ("ne", A.NE), ("eq", A.EQ)):
        shapes["cc_" + name] = one(Filter(Scan(e), op, 0, 1), U2)                                # h(X,Y) :- e(X,Y), X op Y
        shapes["const_" + name] = one(Filter(Scan(e), op, 1, 37, True), U2)                      # h(X,Y) :- e(X,Y), Y op 37
    # recursion with a filter inside the recursive rule: h(X,Z) :- h(X,Y), e(Y,Z), X < Z
    base = CompiledRule("h", Scan(e), U2)
    rec = CompiledRule("h", Project(Filter(Join(Scan(h), Scan(e), [1], [0]), A.LT, 0, 3), [0, 3]), U2)
    shapes["rec_filter"] = ExecutionPlan([Scc(0, True, [base, rec])], ids)
    return shapes


@pytest.mark.parametrize("name", sorted(_plans()))
@pytest.mark.parametrize("rows,bits", [(0, 6), (1, 6), (300, 6), (5000, 9)])
def test_shape_against_oracle(oracle, name, rows, bits):
    plan = _plans()[name]
    inputs = {"e": _rel(rows, 2, bits, 11), "n": _rel(max(rows // 3, 0), 1, bits, 29)}
    want, ex = oracle.run_program(plan, inputs, ["h"])
    for flags in (0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        got, stats = run_program(p, plan, inputs, ["h"])
        assert len(got["h"]) == len(want["h"])
        for g, w in zip(got["h"], want["h"]):
            assert np.array_equal(g, w), f"{name} rows={rows} flags={flags}"
        assert stats["candidate_tuples"] == ex.candidates
        p.close()
