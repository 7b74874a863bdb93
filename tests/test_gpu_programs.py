"""Parity of the CUDA fixpoint (through the C ABI) with the CPU oracle on seeded inputs."""
import numpy as np
import pytest

from xlog_b200 import programs, workloads
from xlog_b200.executor import run_program
from xlog_b200.provider import KernelProvider

pytestmark = pytest.mark.gpu


def _check(provider, oracle, plan, inputs, outputs):
    got, stats = run_program(provider, plan, inputs, outputs)
    want, ex = oracle.run_program(plan, inputs, outputs)
    for o in outputs:
        assert len(got[o]) == len(want[o])
        for g, w in zip(got[o], want[o]):
            assert g.dtype == w.dtype
            assert np.array_equal(g, w), f"{o}: CUDA result differs from the oracle"
    assert stats["candidate_tuples"] == ex.candidates
    return got, stats


def fresh():
    return KernelProvider(device=0)


@pytest.mark.parametrize("nodes,edges,seed", [(10, 20, 1), (300, 900, 7), (2000, 10000, None)])
def test_transitive_closure_uniform(oracle, nodes, edges, seed):
    c0, c1 = workloads.uniform_digraph(nodes, edges, seed)
    p = fresh()
    _check(p, oracle, programs.transitive_closure(), {"edge": [c0, c1]}, ["reach"])
    p.close()


@pytest.mark.parametrize("builder", [programs.transitive_closure_left_linear, programs.transitive_closure_nonlinear,
                                     programs.transitive_closure_swapped_head])
def test_transitive_closure_variants(oracle, builder):
    c0, c1 = workloads.uniform_digraph(200, 500, 3)
    p = fresh()
    _check(p, oracle, builder(), {"edge": [c0, c1]}, ["reach"])
    p.close()


def test_reach_from_source_rmat(oracle):
    c0, c1 = workloads.rmat_graph(14, 16)
    p = fresh()
    got, _ = _check(p, oracle, programs.reach_from_source(0), {"edge": [c0, c1]}, ["r"])
    assert len(got["r"][0]) > 1000
    p.close()


def test_same_generation_tree(oracle):
    c0, c1, _ = workloads.tree_dag(1500, 0.05, 5)
    p = fresh()
    _check(p, oracle, programs.same_generation(), {"edge": [c0, c1]}, ["sg"])
    p.close()


def test_andersen_small(oracle):
    inp = workloads.andersen_program(0.0002)
    p = fresh()
    _check(p, oracle, programs.andersen(), {k: list(v) for k, v in inp.items()}, ["pt"])
    p.close()


def test_rmat_dag_closure(oracle):
    c0, c1 = workloads.rmat_dag(12, 8)
    p = fresh()
    _check(p, oracle, programs.transitive_closure(), {"edge": [c0, c1]}, ["reach"])
    p.close()


def test_chunked_join_matches_unchunked(oracle):
    c0, c1 = workloads.uniform_digraph(300, 900, 7)
    p = KernelProvider(device=0, join_chunk_tuples=5000)
    got, stats = run_program(p, programs.transitive_closure(), {"edge": [c0, c1]}, ["reach"])
    want, _ = oracle.run_program(programs.transitive_closure(), {"edge": [c0, c1]}, ["reach"])
    assert all(np.array_equal(g, w) for g, w in zip(got["reach"], want["reach"]))
    p.close()


# ---- the reference's end-to-end fixtures -------------------------------------------------------
from test_oracle_golden import PROGS, program_inputs, rows_of  # noqa: E402


@pytest.mark.parametrize("case", PROGS["programs"], ids=lambda c: c["name"])
def test_program_kat(case):
    plan, facts, out = program_inputs(case)
    p = fresh()
    got, _ = run_program(p, plan, facts, [out])
    assert rows_of(got[out]) == case["expected"], case["cite"]
    p.close()


def test_novel_step_emits_sorted_unique_rows(provider):
    from test_oracle_golden import cols_of
    ns = PROGS["novel_step"]
    t2 = ["u32", "u32"]
    mk = lambda rows: provider.create_buffer_from_slices(cols_of(rows, t2))
    joined = provider.download(provider.hash_join_v2(mk(ns["delta"]), mk(ns["edge"]), [1], [0]))
    cand = provider.create_buffer_from_slices([joined[0], joined[3]])
    novel = provider.diff_gpu(cand, mk(ns["full"]))
    assert rows_of(provider.download(novel)) == ns["expected"] and novel.is_canonical()


def test_iteration_limit_is_an_error_with_the_reference_message():
    from xlog_b200.lib import XlbError
    from xlog_b200 import _abi as A
    c0 = np.arange(0, 50, dtype=np.uint32)
    p = KernelProvider(device=0, max_iterations=3)
    with pytest.raises(XlbError) as e:
        run_program(p, programs.transitive_closure(), {"edge": [c0, c0 + 1]}, ["reach"])
    assert e.value.status == A.ERR_ITER_LIMIT and "iteration limit (3) exceeded" in e.value.message
    p.close()


def test_missing_input_relation_is_reported():
    from xlog_b200.lib import XlbError
    from xlog_b200 import _abi as A
    p = fresh()
    with pytest.raises(XlbError) as e:
        run_program(p, programs.transitive_closure(), {}, ["reach"])
    assert e.value.status == A.ERR_NOT_FOUND and "Missing relation: edge" in e.value.message
    p.close()


def test_rerun_after_new_facts_extends_the_fixpoint(oracle):
    """Running the plan again after an input grew continues from the stored relation, as the
    reference's seeding pass does (executor/recursive.rs:525-566)."""
    from xlog_b200.executor import Executor
    c0, c1 = workloads.uniform_digraph(150, 400, 5)
    plan = programs.transitive_closure()
    p = fresh()
    ex = Executor(p)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    ex.put_relation("edge", p.create_buffer_from_slices([c0[:300], c1[:300]]))
    ex.execute_plan(plan)
    ex.put_relation("edge", p.create_buffer_from_slices([c0, c1]))
    ex.execute_plan(plan)
    got = p.download(ex.get("reach"))
    want, _ = oracle.run_program(plan, {"edge": [c0, c1]}, ["reach"])
    assert all(np.array_equal(g, w) for g, w in zip(got, want["reach"]))
    p.close()


def test_rules_on_several_ranks_outside_the_packed_scope_are_refused_not_miscomputed():
    """The general evaluator (three and more live columns) runs on one rank; a context that belongs to a
    group of ranks refuses such a rule with a message instead of computing on a shard."""
    from xlog_b200.lib import XlbError
    from xlog_b200 import _abi as A
    from xlog_b200.plan import CompiledRule, ExecutionPlan, Join, Project, Scan, Scc
    body = Project(Join(Scan(0), Scan(0), [1], [0]), [0, 1, 3])
    plan = ExecutionPlan([Scc(0, False, [CompiledRule("path3", body, (A.U32, A.U32, A.U32))])], {"edge": 0, "path3": 1})
    c0, c1 = workloads.uniform_digraph(50, 200, 2)
    p = fresh()
    p._check(p._lib.xlb_comm_mark_aborted_for_test(p._ctx))      # records a world of two ranks; no peer is involved
    with pytest.raises(XlbError) as e:
        run_program(p, plan, {"edge": [c0, c1]}, ["path3"])
    assert e.value.status == A.ERR_UNSUPPORTED and "one rank" in e.value.message
    p.close()


def test_triangle_body_with_a_closing_atom(oracle):
    """tri(X) :- edge(X,Y), edge(Y,Z), edge(Z,X): the last atom has both columns bound and is
    evaluated as a membership test on the row index; also as a recursive rule's filter atom."""
    from xlog_b200.plan import CompiledRule, ExecutionPlan, Join, Project, Scan, Scc
    from xlog_b200 import _abi as A
    c0, c1 = workloads.uniform_digraph(300, 4000, 6)
    # columns: X Y | Y Z | Z X  -> join keys (Z, X) against (col0, col1) of the third atom
    body = Project(Join(Join(Scan(0), Scan(0), [1], [0]), Scan(0), [3, 0], [0, 1]), [0])
    plan = ExecutionPlan([Scc(0, False, [CompiledRule("tri", body, (A.U32,))])], {"edge": 0, "tri": 1})
    want, _ = oracle.run_program(plan, {"edge": [c0, c1]}, ["tri"])
    assert len(want["tri"][0]) > 50
    for flags in (0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        got, _ = run_program(p, plan, {"edge": [c0, c1]}, ["tri"])
        assert all(np.array_equal(g, w) for g, w in zip(got["tri"], want["tri"]))
        p.close()
    # recursive use: reach restricted to pairs that are also edges of a second relation
    base = CompiledRule("r", Scan(0), (A.U32, A.U32))
    rec = CompiledRule("r", Project(Join(Join(Scan(2), Scan(0), [1], [0]), Scan(1), [0, 3], [0, 1]), [0, 3]), (A.U32, A.U32))
    plan2 = ExecutionPlan([Scc(0, True, [base, rec])], {"edge": 0, "allow": 1, "r": 2})
    a0, a1 = workloads.uniform_digraph(300, 30000, 9)
    inputs = {"edge": [c0[:1500], c1[:1500]], "allow": [a0, a1]}
    want2, _ = oracle.run_program(plan2, inputs, ["r"])
    p = fresh()
    got2, _ = run_program(p, plan2, inputs, ["r"])
    assert all(np.array_equal(g, w) for g, w in zip(got2["r"], want2["r"]))
    assert len(got2["r"][0]) > 1500
    p.close()


@pytest.mark.parametrize("name", ["tc", "reach", "sg"])
def test_dense_route_on_and_off_agree(oracle, name):
    """Small-domain fixpoints take the bitmap route by default; with the kill switch they take the
    sort / merge route.  Both must give the oracle's result (the reference pins its own fast route
    the same way: crates/xlog-integration/tests/test_factorized_delta_e2e.rs:280-308)."""
    from xlog_b200 import _abi as A
    if name == "tc":
        c0, c1 = workloads.uniform_digraph(500, 2000, 4)
        plan, inputs, out = programs.transitive_closure(), {"edge": [c0, c1]}, "reach"
    elif name == "reach":
        c0, c1 = workloads.rmat_graph(13, 16)
        plan, inputs, out = programs.reach_from_source(0), {"edge": [c0, c1]}, "r"
    else:
        c0, c1, _ = workloads.tree_dag(1200, 0.05, 8)
        plan, inputs, out = programs.same_generation(), {"edge": [c0, c1]}, "sg"
    want, _ = oracle.run_program(plan, inputs, [out])
    results = []
    for flags in (0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        p.profile_enable("*")
        got, _ = run_program(p, plan, inputs, [out])
        prof = p.profile_read()
        used_dense = "dense_mark" in prof or "expand_mark" in prof
        assert used_dense == (flags == 0), "the route taken is not the one asked for"
        assert all(np.array_equal(g, w) for g, w in zip(got[out], want[out]))
        p.close()


def test_stratified_negation_and_union_body(oracle):
    """Anti join against a lower stratum and a Union at the top of a rule body."""
    from test_oracle_golden import stratified_case
    plan, inputs, reach, unreach = stratified_case()
    p = fresh()
    got, _ = run_program(p, plan, inputs, ["r", "un", "either"])
    want, _ = oracle.run_program(plan, inputs, ["r", "un", "either"])
    for name in ("r", "un", "either"):
        assert np.array_equal(got[name][0], want[name][0])
    assert got["un"][0].tolist() == sorted(unreach)
    p.close()


def test_the_tuple_whose_mixed_word_is_the_empty_mark(oracle):
    """The hash set of a wide head stores mix64(tuple) and marks empty slots with all ones; exactly one
    tuple mixes to that word and is kept in a flag of its own.  It must be derived once, however
    often it is a candidate, and must not be lost."""
    from xlog_b200 import _abi as A
    from xlog_b200.dist import mix64
    M = (1 << 64) - 1

    def unmix(x):
        x ^= x >> 33
        x = (x * pow(0xC4CEB9FE1A85EC53, -1, 1 << 64)) & M
        x ^= x >> 33
        x = (x * pow(0xFF51AFD7ED558CCD, -1, 1 << 64)) & M
        x ^= x >> 33
        return x

    k0 = unmix(M)
    assert int(mix64(np.array([k0], np.uint64))[0]) == M
    a, b = k0 >> 32, k0 & 0xFFFFFFFF
    # the edge (a, b) three times, a way around it (a -> 7 -> b is not an edge pair that gives (a, b) again, but
    # (9, a) and (a, b) give (9, b)), and unrelated edges; ids this large never fit a bitmap
    c0 = np.array([a, a, a, 9, b, 5, 9], np.uint32)
    c1 = np.array([b, b, b, a, 11, 6, 11], np.uint32)
    plan = programs.transitive_closure()
    want, ex = oracle.run_program(plan, {"edge": [c0, c1]}, ["reach"])
    for flags in (0, A.FLAG_NO_TUPLE_SET):
        p = KernelProvider(device=0, flags=flags)
        p.profile_enable("*")
        got, stats = run_program(p, plan, {"edge": [c0, c1]}, ["reach"])
        used_set = "hset_insert" in p.profile_read()
        assert used_set == (flags == 0)
        assert all(np.array_equal(g, w) for g, w in zip(got["reach"], want["reach"]))
        assert (a, b) in set(zip(got["reach"][0].tolist(), got["reach"][1].tolist()))
        assert stats["candidate_tuples"] == ex.candidates
        p.close()
