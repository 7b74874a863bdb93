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
