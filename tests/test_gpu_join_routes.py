"""The routes a join step can take (scan join, counting index, sorted index with a hash table) and
the bitmap that carries a head relation across iterations, each pinned against the CPU oracle:
same tuples, same candidate count, whichever route ran."""
import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import programs
from xlog_b200.executor import Executor, run_program
from xlog_b200.plan import CompiledRule, ExecutionPlan, Join, Project, Scan, Scc
from xlog_b200.provider import KernelProvider
from xlog_b200.workloads import shuffle_rows, splitmix64

pytestmark = pytest.mark.gpu
U1, U2 = (A.U32,), (A.U32, A.U32)


def _same(got, want, what=""):
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert np.array_equal(g, w), what


def _chain(n, extra, seed):
    """0 -> 1 -> ... -> n-1 plus `extra` pseudo-random backward edges (no short cuts: node k is
    first reached in iteration k), rows shuffled."""
    a = np.arange(n - 1, dtype=np.uint32)
    x0 = (splitmix64(seed, 0, extra) % np.uint64(n)).astype(np.uint32)
    x1 = (splitmix64(seed + 1, 0, extra) % np.uint64(n)).astype(np.uint32)
    x0, x1 = np.maximum(x0, x1), np.minimum(x0, x1)
    c0, c1 = np.concatenate([a, x0]), np.concatenate([a + 1, x1])
    return shuffle_rows([c0, c1], seed + 2)


@pytest.mark.parametrize("flags", [0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET])
def test_long_chain_goes_from_scans_to_an_index(oracle, flags):
    # 80 iterations: more than the scans a relation is given before its index is built
    c0, c1 = _chain(81, 40, 5)
    plan = programs.reach_from_source(0)
    p = KernelProvider(device=0, flags=flags)
    got, stats = run_program(p, plan, {"edge": [c0, c1]}, ["r"])
    want, ex = oracle.run_program(plan, {"edge": [c0, c1]}, ["r"])
    _same(got["r"], want["r"])
    assert stats["candidate_tuples"] == ex.candidates
    assert stats["iterations"] >= 80
    p.close()


def test_sorted_input_gets_its_index_after_three_scans(oracle):
    # the same program over a relation certified sorted and unique (the output of dedup)
    c0, c1 = _chain(30, 25, 9)
    plan = programs.reach_from_source(0)
    p = KernelProvider(device=0)
    ex = Executor(p)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    edge = p.dedup(p.sort(p.create_buffer_from_slices([c0, c1]), [0, 1]), [0, 1])
    assert edge.is_canonical()
    ex.put_relation("edge", edge)
    stats = ex.execute_plan(plan)
    got = p.download(ex.get("r"))
    want, _ = oracle.run_program(plan, {"edge": [c0, c1]}, ["r"])
    _same(got, want["r"])
    # the oracle saw the rows with their duplicates: compare candidates on the deduplicated input
    d0, d1 = p.download(edge)
    _, oex = oracle.run_program(plan, {"edge": [d0, d1]}, ["r"])
    assert stats["candidate_tuples"] == oex.candidates
    p.close()


def test_duplicate_rows_count_once_per_row_on_every_route(oracle):
    c0, c1 = _chain(40, 60, 3)
    c0, c1 = np.concatenate([c0, c0[:30]]), np.concatenate([c1, c1[:30]])  # 30 rows twice
    plan = programs.reach_from_source(0)
    want, ex = oracle.run_program(plan, {"edge": [c0, c1]}, ["r"])
    for flags in (0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        got, stats = run_program(p, plan, {"edge": [c0, c1]}, ["r"])
        _same(got["r"], want["r"], f"flags={flags}")
        assert stats["candidate_tuples"] == ex.candidates
        p.close()


def test_ids_beyond_the_dense_domain_take_the_hash_route(oracle):
    # node ids around 2^30: no bitmap of keys or tuples is possible, the sorted index with its hash
    # table serves the joins and sort + merge the set difference
    c0, c1 = _chain(50, 80, 13)
    big = np.uint32(1 << 30)
    c0, c1 = c0 * np.uint32(7919) + big, c1 * np.uint32(7919) + big
    for plan, out in ((programs.reach_from_source(int(big)), "r"), (programs.transitive_closure(), "reach")):
        p = KernelProvider(device=0)
        got, stats = run_program(p, plan, {"edge": [c0, c1]}, [out])
        want, ex = oracle.run_program(plan, {"edge": [c0, c1]}, [out])
        _same(got[out], want[out])
        assert stats["candidate_tuples"] == ex.candidates
        p.close()


def _two_source_plan():
    """h(X) :- a(X).   h(Y) :- h(X), b(X,Y).   `a` holds small ids, `b` reaches large ones: the
    bitmap of h is first sized by `a` and has to widen when the recursive rule runs."""
    ids = {"a": 0, "b": 1, "h": 2}
    base = CompiledRule("h", Scan(ids["a"]), U1)
    rec = CompiledRule("h", Project(Join(Scan(ids["h"]), Scan(ids["b"]), [0], [0]), [2]), U1)
    return ExecutionPlan([Scc(0, True, [base, rec])], ids)


@pytest.mark.parametrize("flags", [0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET])
def test_head_bitmap_widens_with_the_domain(oracle, flags):
    a = [np.array([1, 2, 3, 5], dtype=np.uint32)]
    b0 = np.array([1, 2, 3, 900, 70000, 5, 1 << 20], dtype=np.uint32)
    b1 = np.array([900, 70000, 3, 1 << 20, 12, 5, 2], dtype=np.uint32)
    plan = _two_source_plan()
    p = KernelProvider(device=0, flags=flags)
    got, stats = run_program(p, plan, {"a": a, "b": [b0, b1]}, ["h"])
    want, ex = oracle.run_program(plan, {"a": a, "b": [b0, b1]}, ["h"])
    _same(got["h"], want["h"])
    assert stats["candidate_tuples"] == ex.candidates
    p.close()


def test_head_that_already_holds_rows_is_not_derived_again(oracle):
    # h is put into the store with rows before the plan runs: they are in `full` from the start and
    # must come out once, whether the bitmap or the merge path subtracts them
    a = [np.array([4, 9], dtype=np.uint32)]
    b0 = np.array([4, 9, 11, 12], dtype=np.uint32)
    b1 = np.array([11, 12, 4, 30], dtype=np.uint32)
    h0 = [np.array([30, 11, 11, 500], dtype=np.uint32)]  # unsorted, with a duplicate
    plan = _two_source_plan()
    want, ex = oracle.run_program(plan, {"a": a, "b": [b0, b1], "h": h0}, ["h"])
    for flags in (0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        got, _ = run_program(p, plan, {"a": a, "b": [b0, b1], "h": h0}, ["h"])
        _same(got["h"], want["h"], f"flags={flags}")
        p.close()


def test_scan_join_at_bench_shape_matches_the_index_route():
    # a power-law graph large enough for whole 16-byte tiles and many blocks; the two routes must
    # agree with each other on tuples and candidate count (the oracle covers smaller cases)
    from xlog_b200 import workloads
    c0, c1 = workloads.rmat_graph(16, 16)
    plan = programs.reach_from_source(0)
    res = []
    for flags in (0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        got, stats = run_program(p, plan, {"edge": [c0, c1]}, ["r"])
        res.append((got["r"], stats["candidate_tuples"], stats["derived_tuples"]))
        p.close()
    _same(res[0][0], res[1][0])
    assert res[0][1:] == res[1][1:]
    assert np.all(np.diff(res[0][0][0].astype(np.int64)) > 0)
