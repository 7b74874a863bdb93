"""Parity at the full size of the benchmark configurations that fit one GPU, through checks that
do not need the CPU oracle to finish a whole fixpoint: an independent breadth-first search
(scipy's, on a CSR matrix) for the reachable set of config 2, closure and sortedness properties,
idempotence, and agreement of the two routes."""
import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import programs, workloads
from xlog_b200.executor import Executor, run_program
from xlog_b200.provider import KernelProvider

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def c2_edges():
    return workloads.rmat_graph(20, 16)     # 16 086 179 edges, rows in a seeded pseudo-random order


def test_config2_full_size_equals_an_independent_bfs(c2_edges):
    from scipy.sparse import csr_matrix
    from scipy.sparse.csgraph import breadth_first_order
    c0, c1 = c2_edges
    n = 1 << 20
    assert len(c0) == 16_086_179
    graph = csr_matrix((np.ones(len(c0), np.int8), (c0.astype(np.int64), c1.astype(np.int64))), shape=(n, n))
    order = breadth_first_order(graph, 0, directed=True, return_predecessors=False)
    # r holds what is reachable in one step or more: the source itself only if a cycle leads back
    reach = np.sort(order[1:].astype(np.uint32))
    back = np.isin(0, c1[np.isin(c0, order)])
    want = np.sort(np.append(reach, np.uint32(0))) if back else reach

    plan = programs.reach_from_source(0)
    results = []
    for flags in (0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        got, stats = run_program(p, plan, {"edge": [c0, c1]}, ["r"])
        results.append((got["r"][0], stats["candidate_tuples"], stats["iterations"]))
        p.close()
    for r, cand, _ in results:
        assert r.dtype == np.uint32 and np.array_equal(r, want)          # the same set, sorted, no repeats
    assert results[0][1] == results[1][1] == 15_979_774                   # both routes count the same join output
    # closure: no edge leaves the set
    inside = np.zeros(n, bool)
    inside[want] = True
    assert inside[c1[inside[c0]]].all() and inside[c1[c0 == 0]].all()


def test_config2_full_size_is_idempotent(c2_edges):
    # running the plan again over its own result derives nothing new
    c0, c1 = c2_edges
    plan = programs.reach_from_source(0)
    p = KernelProvider(device=0)
    ex = Executor(p)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    ex.put_relation("edge", p.create_buffer_from_slices([c0, c1]))
    s1 = ex.execute_plan(plan)
    first = p.download(ex.get("r"))[0]
    s2 = ex.execute_plan(plan)
    again = p.download(ex.get("r"))[0]
    assert np.array_equal(first, again) and s1["derived_tuples"] == len(first)
    assert s2["iterations"] <= 2
    p.close()


def _closure_bitsets(c0, c1, n):
    """Transitive closure of a DAG whose edges all lead from a lower to a higher id, as one bit row
    per vertex, filled from the highest id down: a row is the OR of its successors' rows plus the
    successors themselves.  Shares nothing with the library or with the CPU port of the engine."""
    words = (n + 63) // 64
    rows = np.zeros((n, words), dtype=np.uint64)
    order = np.argsort(c0, kind="stable")
    dst = c1[order]
    starts = np.searchsorted(c0[order], np.arange(n + 1))
    for v in range(n - 1, -1, -1):
        kids = dst[starts[v]:starts[v + 1]]
        if len(kids):
            row = np.bitwise_or.reduce(rows[kids], axis=0)
            np.bitwise_or.at(row, kids >> 6, np.uint64(1) << (kids & 63).astype(np.uint64))
            rows[v] = row
    return rows


@pytest.mark.parametrize("scale,want_rows", [(14, None), (16, 178_519_106)])
def test_closure_of_the_banded_dag_at_middle_scales(scale, want_rows):
    # the secondary workload of the benchmark at 2^14 and 2^16 vertices: the count, the per-source
    # counts and a digest of the rows are checked against bit rows computed on the host, and the
    # three routes of the engine (bitmap, hash set, sort) must deliver the same sorted relation
    from xlog_b200 import digest
    n = 1 << scale
    c0, c1 = workloads.rmat_dag(scale, 8)
    assert (c0 < c1).all()
    rows = _closure_bitsets(c0, c1, n)
    per_source = np.bitwise_count(rows).sum(axis=1, dtype=np.int64)
    total = int(per_source.sum())
    if want_rows is not None:
        assert total == want_rows
    plan = programs.transitive_closure()
    digests = []
    for flags in (0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        ex = Executor(p)
        for name, rid in plan.rel_ids.items():
            ex.register_relation(rid, name)
        ex.put_relation("edge", p.create_buffer_from_slices([c0, c1]))
        stats = ex.execute_plan(plan)
        assert stats["derived_tuples"] == total
        digests.append(p.checksum(ex.get("reach")))
        if flags == 0 or scale == 14:
            a, b = p.download(ex.get("reach"))
            assert len(a) == total
            key = (a.astype(np.uint64) << np.uint64(32)) | b
            assert (key[1:] > key[:-1]).all()                                   # sorted, no repeats
            assert np.array_equal(np.bincount(a, minlength=n), per_source)      # as many rows per source
            hit = (rows[a, b >> 6] >> (b & 63).astype(np.uint64)) & np.uint64(1)
            assert hit.all()                                                    # and every one of them reachable
            assert digest.result_checksum([a, b]) == digests[-1]                    # the device digest is of these rows
            del a, b, key, hit
        p.close()
    assert digests[0] == digests[1] == digests[2]
