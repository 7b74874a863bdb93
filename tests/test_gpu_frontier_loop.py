"""The frontier loop of a one-column head (``r(Y) :- r(X), rel(X, Y)``): the stored relation is
streamed over as columns or as packed rows, rows whose key the head already holds drop out of the
later scans, and the general loop takes over when the relation has been streamed over too often.
Every case is compared with the CPU oracle: result and candidate count."""
import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import programs, workloads
from xlog_b200.executor import Executor, run_program
from xlog_b200.plan import CompiledRule, ExecutionPlan, Filter, Join, Project, Scan, Scc
from xlog_b200.provider import KernelProvider

pytestmark = pytest.mark.gpu


def _same_as_oracle(oracle, plan, inputs, outs, flags=0):
    p = KernelProvider(device=0, flags=flags)
    got, stats = run_program(p, plan, inputs, outs)
    p.close()
    want, ex = oracle.run_program(plan, inputs, outs)
    for o in outs:
        assert len(got[o]) == len(want[o])
        for g, w in zip(got[o], want[o]):
            assert g.dtype == w.dtype and np.array_equal(g, w), f"{o}: CUDA result differs from the oracle"
    assert stats["candidate_tuples"] == ex.candidates
    return got, stats


def reach_backwards(target: int) -> ExecutionPlan:
    """r(X) :- edge(X, target).  r(X) :- r(Y), edge(X, Y).   (the join runs on the second column)"""
    ids = {"edge": 0, "r": 1}
    base = CompiledRule("r", Project(Filter(Scan(0), A.EQ, 1, target, True), [0]), (A.U32,))
    rec = CompiledRule("r", Project(Join(Scan(1), Scan(0), [0], [1]), [1]), (A.U32,))
    return ExecutionPlan([Scc(0, True, [base, rec])], ids)


@pytest.mark.parametrize("rows", [1, 3, 7, 2047, 2048, 2049, 4099, 20001])
def test_row_counts_around_the_tile_size(oracle, rows):
    # whole tiles take 16-byte loads, the last partial tile scalar ones; the lists of rows still of
    # use are written by whole tiles too
    c0, c1 = workloads.uniform_digraph(max(8, rows // 3), 2 * rows + 8, 11)
    c0, c1 = c0[:rows].copy(), c1[:rows].copy()
    assert len(c0) == rows
    c0[0] = 0                                                      # the source has an edge
    _same_as_oracle(oracle, programs.reach_from_source(0), {"edge": [c0, c1]}, ["r"])


@pytest.mark.parametrize("flags", [0, A.FLAG_NO_DENSE])
def test_join_on_the_second_column(oracle, flags):
    c0, c1 = workloads.rmat_graph(13, 8)
    target = int(c1[0])
    got, _ = _same_as_oracle(oracle, reach_backwards(target), {"edge": [c0, c1]}, ["r"], flags)
    assert len(got["r"][0]) > 100


def test_keys_far_outside_the_heads_domain(oracle):
    # sources that nothing leads to carry ids near 2^32: the head's domain is sized by the values
    # it can take (second column), so those rows can never match and must not disturb the bitmaps
    c0, c1 = workloads.rmat_graph(12, 8)
    far = np.arange(200, dtype=np.uint32) + np.uint32(0xFFFFFF00 - 200)
    c0 = np.concatenate([c0, far])
    c1 = np.concatenate([c1, np.arange(200, dtype=np.uint32)])
    _same_as_oracle(oracle, programs.reach_from_source(0), {"edge": [c0, c1]}, ["r"])


def test_a_long_path_hands_over_to_the_general_loop(oracle):
    # 60 iterations: after a dozen scans the loop stops streaming and the general loop (which packs
    # the relation and builds an index) finishes from the stored state
    n = 60
    chain0 = np.arange(n, dtype=np.uint32)
    chain1 = chain0 + 1
    e0, e1 = workloads.uniform_digraph(400, 3000, 5)
    e0, e1 = e0 + np.uint32(1000), e1 + np.uint32(1000)              # a component the source does not reach
    c0 = np.concatenate([chain0, e0, np.array([n], np.uint32)])
    c1 = np.concatenate([chain1, e1, np.array([1000], np.uint32)])   # ... until the end of the path leads into it
    got, stats = _same_as_oracle(oracle, programs.reach_from_source(0), {"edge": [c0, c1]}, ["r"])
    assert stats["iterations"] >= 60


def test_a_relation_packed_by_an_earlier_component_is_streamed_as_rows(oracle):
    # two(X, Z) :- edge(X, Y), edge(Y, Z) runs first and packs `edge`; the reachability component
    # then finds the packed rows and streams over those
    ids = {"edge": 0, "two": 1, "r": 2}
    two = CompiledRule("two", Project(Join(Scan(0), Scan(0), [1], [0]), [0, 3]), (A.U32, A.U32))
    base = CompiledRule("r", Project(Filter(Scan(0), A.EQ, 0, 0, True), [1]), (A.U32,))
    rec = CompiledRule("r", Project(Join(Scan(2), Scan(0), [0], [0]), [2]), (A.U32,))
    plan = ExecutionPlan([Scc(0, False, [two]), Scc(1, True, [base, rec])], ids)
    c0, c1 = workloads.rmat_graph(11, 6)
    _same_as_oracle(oracle, plan, {"edge": [c0, c1]}, ["two", "r"])


def test_running_the_plan_again_finds_the_columns_bound_known(oracle):
    c0, c1 = workloads.rmat_graph(13, 16)
    plan = programs.reach_from_source(0)
    want, ex = oracle.run_program(plan, {"edge": [c0, c1]}, ["r"])
    p = KernelProvider(device=0)
    e = Executor(p)
    for name, rid in plan.rel_ids.items():
        e.register_relation(rid, name)
    e.put_relation("edge", p.create_buffer_from_slices([c0, c1]))
    s1 = e.execute_plan(plan)
    first = p.download(e.get("r"))[0]
    s2 = e.execute_plan(plan)
    again = p.download(e.get("r"))[0]
    assert np.array_equal(first, want["r"][0]) and np.array_equal(again, first)
    assert s1["candidate_tuples"] == ex.candidates and s2["iterations"] <= 2
    # the columns handed in are as they were
    b0, b1 = p.download(e.get("edge"))
    assert np.array_equal(b0, c0) and np.array_equal(b1, c1)
    p.close()


def test_full_size_scan_shrinks_with_the_rows_left(oracle):
    # the profile of the run says how many bytes the scans moved: far fewer than one full stream
    # over the relation per iteration
    c0, c1 = workloads.rmat_graph(16, 16)
    plan = programs.reach_from_source(0)
    p = KernelProvider(device=0, profile=True)
    p.profile_enable("*")
    got, stats = run_program(p, plan, {"edge": [c0, c1]}, ["r"])
    prof = p.profile_read()
    p.close()
    want, ex = oracle.run_program(plan, {"edge": [c0, c1]}, ["r"])
    assert np.array_equal(got["r"][0], want["r"][0]) and stats["candidate_tuples"] == ex.candidates
    scans = prof["scan_join_mark"]
    assert scans["launches"] >= stats["iterations"] - 1
    assert 0 < scans["bytes"] < 0.8 * stats["iterations"] * len(c0) * 8
