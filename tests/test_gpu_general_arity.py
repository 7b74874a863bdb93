"""Rules the packed pipelines do not take: more than two live columns, relations and heads of three
and more columns, two-column join keys as real joins, a Union below the top of a body, a semi /
anti join against a subtree.  They run on the general, node-by-node evaluator
(xlog_b200/csrc/xlb_tree.cu), which follows the reference's execute_node
(crates/xlog-runtime/src/executor/node_dispatch.rs:98-319).  Every result is compared with the CPU
oracle bit for bit, the candidate count included; XLB_FLAG_GENERAL_ONLY also sends the ordinary
two-column programs through it, so that the two engines check each other.
"""
import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import programs, workloads
from xlog_b200.executor import run_program
from xlog_b200.plan import CompiledRule, Diff, Distinct, ExecutionPlan, Filter, Join, Project, Scan, Scc, Union
from xlog_b200.provider import KernelProvider

pytestmark = pytest.mark.gpu
U3 = (A.U32, A.U32, A.U32)


def _check(oracle, plan, inputs, outputs, flags=0, **kw):
    p = KernelProvider(device=0, flags=flags, **kw)
    try:
        got, stats = run_program(p, plan, inputs, outputs)
        want, ex = oracle.run_program(plan, inputs, outputs)
        for o in outputs:
            assert len(got[o]) == len(want[o])
            for g, w in zip(got[o], want[o]):
                assert g.dtype == w.dtype and np.array_equal(g, w), f"{o}: CUDA result differs from the oracle"
        assert stats["candidate_tuples"] == ex.candidates
        assert stats["iterations"] == ex.iterations
        return got, stats
    finally:
        p.close()


def test_three_column_head_runs(oracle):
    """path3(X,Y,Z) :- edge(X,Y), edge(Y,Z): three live columns (was refused before the general evaluator)."""
    body = Project(Join(Scan(0), Scan(0), [1], [0]), [0, 1, 3])
    plan = ExecutionPlan([Scc(0, False, [CompiledRule("path3", body, U3)])], {"edge": 0, "path3": 1})
    c0, c1 = workloads.uniform_digraph(50, 200, 2)
    got, _ = _check(oracle, plan, {"edge": [c0, c1]}, ["path3"])
    assert len(got["path3"]) == 3 and len(got["path3"][0]) > 200


def test_two_column_join_key_inside_a_plan(oracle):
    """The reference's multi-column join case (crates/xlog-cuda/tests/join_v2_tests.rs:304-353) as a
    rule: m(A,B,P,V) :- l(A,B,P), r(A,B,V)."""
    left = [np.array(x, np.uint32) for x in ([1, 1, 2], [10, 20, 10], [100, 200, 300])]
    right = [np.array(x, np.uint32) for x in ([1, 2, 1], [10, 10, 20], [1000, 2000, 3000])]
    body = Project(Join(Scan(0), Scan(1), [0, 1], [0, 1]), [0, 1, 2, 5])
    plan = ExecutionPlan([Scc(0, False, [CompiledRule("m", body, (A.U32,) * 4)])], {"l": 0, "r": 1, "m": 2})
    got, _ = _check(oracle, plan, {"l": left, "r": right}, ["m"])
    rows = sorted(zip(*[c.tolist() for c in got["m"]]))
    assert rows == [(1, 10, 100, 1000), (1, 20, 200, 3000), (2, 10, 300, 2000)]


def test_triangle_listing(oracle):
    """tri(X,Y,Z) :- edge(X,Y), edge(Y,Z), edge(Z,X): a three-column head over a two-column key join."""
    c0, c1 = workloads.uniform_digraph(200, 2500, 6)
    body = Project(Join(Join(Scan(0), Scan(0), [1], [0]), Scan(0), [3, 0], [0, 1]), [0, 1, 3])
    plan = ExecutionPlan([Scc(0, False, [CompiledRule("tri", body, U3)])], {"edge": 0, "tri": 1})
    got, _ = _check(oracle, plan, {"edge": [c0, c1]}, ["tri"])
    assert len(got["tri"][0]) > 10


def test_recursive_rule_with_three_live_columns(oracle):
    """walk(X,Y,Z) :- edge(X,Y), edge(Y,Z).   walk(X,Y,Z) :- walk(X,Y,W), edge(W,Z).
    (every first hop with everything reachable behind it: a recursive head of three columns)"""
    c0, c1 = workloads.uniform_digraph(60, 150, 4)
    base = CompiledRule("walk", Project(Join(Scan(0), Scan(0), [1], [0]), [0, 1, 3]), U3)
    rec = CompiledRule("walk", Project(Join(Scan(1), Scan(0), [2], [0]), [0, 1, 4]), U3)
    plan = ExecutionPlan([Scc(0, True, [base, rec])], {"edge": 0, "walk": 1})
    got, stats = _check(oracle, plan, {"edge": [c0, c1]}, ["walk"])
    assert stats["iterations"] > 2 and len(got["walk"][0]) > 1000


def test_union_below_the_top_and_anti_join_against_a_subtree(oracle):
    """sym(X,Y): the edges of either direction, filtered afterwards (a Union under a Filter), and
    sink(X): nodes with no outgoing edge (an anti join whose right side is a projection)."""
    c0, c1 = workloads.uniform_digraph(80, 200, 8)
    nodes = np.arange(80, dtype=np.uint32)
    sym = CompiledRule("sym", Filter(Union([Scan(0), Project(Scan(0), [1, 0])]), A.LT, 0, 1), (A.U32, A.U32))
    sink = CompiledRule("sink", Join(Scan(1), Project(Scan(0), [0]), [0], [0], A.JOIN_ANTI), (A.U32,))
    plan = ExecutionPlan([Scc(0, False, [sym]), Scc(1, False, [sink])], {"edge": 0, "node": 1, "sym": 2, "sink": 3})
    got, _ = _check(oracle, plan, {"edge": [c0, c1], "node": [nodes]}, ["sym", "sink"])
    assert set(got["sink"][0].tolist()) == set(nodes.tolist()) - set(c0.tolist())


def test_diff_and_distinct_nodes(oracle):
    """RirNode::Diff (crates/xlog-ir/src/rir.rs:429-434, executed at executor/node_dispatch.rs:264) and
    RirNode::Distinct as plan nodes: one_way(X,Y) = edges without their reverse edge; first(X,Y) = one
    successor per node (the first in stable key order); also a Diff inside a recursive component."""
    c0, c1 = workloads.uniform_digraph(70, 400, 10)
    one_way = CompiledRule("one_way", Diff(Scan(0), Project(Scan(0), [1, 0])), (A.U32, A.U32))
    first = CompiledRule("first", Distinct(Scan(0), [0]), (A.U32, A.U32))
    every = CompiledRule("every", Distinct(Union([Scan(0), Scan(0)])), (A.U32, A.U32))
    plan = ExecutionPlan([Scc(0, False, [one_way]), Scc(1, False, [first]), Scc(2, False, [every])],
                         {"edge": 0, "one_way": 1, "first": 2, "every": 3})
    got, _ = _check(oracle, plan, {"edge": [c0, c1]}, ["one_way", "first", "every"])
    pairs = set(zip(c0.tolist(), c1.tolist()))
    assert set(zip(*[c.tolist() for c in got["one_way"]])) == {p for p in pairs if (p[1], p[0]) not in pairs}
    assert len(got["first"][0]) == len(set(c0.tolist()))
    # reach over the one-way edges only, with the Diff inside the recursive component's base rule
    base = CompiledRule("r", Diff(Scan(0), Project(Scan(0), [1, 0])), (A.U32, A.U32))
    rec = CompiledRule("r", Project(Join(Scan(1), Diff(Scan(0), Project(Scan(0), [1, 0])), [1], [0]), [0, 3]), (A.U32, A.U32))
    plan2 = ExecutionPlan([Scc(0, True, [base, rec])], {"edge": 0, "r": 1})
    _check(oracle, plan2, {"edge": [c0, c1]}, ["r"])


@pytest.mark.parametrize("name", ["tc", "tc_nonlinear", "reach0", "sg", "andersen", "negation"])
def test_general_evaluator_agrees_on_the_two_column_programs(oracle, name):
    c0, c1 = workloads.uniform_digraph(150, 450, 13)
    if name == "tc":
        plan, inputs, outs = programs.transitive_closure(), {"edge": [c0, c1]}, ["reach"]
    elif name == "tc_nonlinear":
        plan, inputs, outs = programs.transitive_closure_nonlinear(), {"edge": [c0, c1]}, ["reach"]
    elif name == "reach0":
        r0, r1 = workloads.rmat_graph(12, 16)
        plan, inputs, outs = programs.reach_from_source(0), {"edge": [r0, r1]}, ["r"]
    elif name == "sg":
        t0, t1, _ = workloads.tree_dag(500, 0.05, 9)
        plan, inputs, outs = programs.same_generation(), {"edge": [t0, t1]}, ["sg"]
    elif name == "andersen":
        plan, inputs, outs = programs.andersen(), {k: list(v) for k, v in workloads.andersen_program(0.0002).items()}, ["pt"]
    else:
        plan = programs.unreachable_nodes(int(c0[0]))
        inputs, outs = {"edge": [c0, c1], "node": [np.arange(150, dtype=np.uint32)]}, ["r", "un", "either"]
    _check(oracle, plan, inputs, outs, flags=A.FLAG_GENERAL_ONLY)


def test_three_typed_columns_through_dictionary_ranks(oracle):
    """hop(X,Y,Z) over u64 ids: the plan runs on 32-bit ranks of one dictionary and the head is
    decoded into its declared types (three columns: the general evaluator under the encoding)."""
    c0, c1 = workloads.uniform_digraph(40, 120, 5)
    big = lambda c: c.astype(np.uint64) * np.uint64(1 << 33) + np.uint64(7)
    U64x3 = (A.U64, A.U64, A.U64)
    body = Project(Join(Scan(0), Scan(0), [1], [0]), [0, 1, 3])
    plan = ExecutionPlan([Scc(0, False, [CompiledRule("hop", body, U64x3)])], {"edge": 0, "hop": 1})
    got, _ = _check(oracle, plan, {"edge": [big(c0), big(c1)]}, ["hop"])
    assert got["hop"][0].dtype == np.uint64 and int(got["hop"][0].min()) >= 7


def test_iteration_limit_in_the_general_evaluator():
    from xlog_b200.lib import XlbError
    c0 = np.arange(0, 40, dtype=np.uint32)
    base = CompiledRule("walk", Project(Join(Scan(0), Scan(0), [1], [0]), [0, 1, 3]), U3)
    rec = CompiledRule("walk", Project(Join(Scan(1), Scan(0), [2], [0]), [0, 1, 4]), U3)
    plan = ExecutionPlan([Scc(0, True, [base, rec])], {"edge": 0, "walk": 1})
    p = KernelProvider(device=0, max_iterations=3)
    with pytest.raises(XlbError) as e:
        run_program(p, plan, {"edge": [c0, c0 + 1]}, ["walk"])
    assert e.value.status == A.ERR_ITER_LIMIT and "iteration limit (3) exceeded" in e.value.message
    p.close()


def test_bool_columns(provider):
    """Full-row dedup of a bool column (crates/xlog-cuda/tests/test_full_row_set_algebra.rs:204-216),
    and a bool payload column carried through sort, difference and join."""
    flags = np.array([1, 0, 1, 0, 1], np.uint8)
    rel = provider.create_buffer_from_slices([flags], [A.BOOL])
    out = provider.download(provider.dedup(rel))
    assert out[0].dtype == np.uint8 and out[0].tolist() == [0, 1]
    ids = np.array([5, 3, 9, 3, 7], np.uint32)
    both = provider.create_buffer_from_slices([ids, flags], [A.U32, A.BOOL])
    s = provider.download(provider.sort(both, [0, 1]))
    assert s[0].tolist() == [3, 3, 5, 7, 9] and s[1].tolist() == [0, 0, 1, 1, 1]
    d = provider.download(provider.diff_gpu(both, provider.create_buffer_from_slices([ids[:2], flags[:2]], [A.U32, A.BOOL])))
    assert list(zip(d[0].tolist(), d[1].tolist())) == [(7, 1), (9, 1)]
    j = provider.download(provider.hash_join_v2(both, provider.create_buffer_from_slices([np.array([3, 7], np.uint32)]), [0], [0]))
    assert sorted(zip(j[0].tolist(), j[1].tolist(), j[2].tolist())) == [(3, 0, 3), (3, 0, 3), (7, 1, 7)]
