"""Seeded generators: determinism and the shape each configuration states."""
import numpy as np

from xlog_b200 import workloads as W


def test_splitmix_slices_agree():
    a = W.splitmix64(9, 0, 1000)
    b = np.concatenate([W.splitmix64(9, 0, 400), W.splitmix64(9, 400, 600)])
    assert np.array_equal(a, b)
    # the published SplitMix64 sequence for seed 0
    z = W.splitmix64(0, 0, 2)
    assert int(z[0]) == 0xE220A8397B1DCDAF and int(z[1]) == 0x6E789E6AA1B965F4


def test_uniform_digraph_config1():
    c0, c1 = W.uniform_digraph()
    assert len(c0) == 10000 and c0.max() < 2000 and c1.max() < 2000
    assert np.all(c0 != c1)
    assert len(np.unique(W.pack_pairs(c0, c1))) == 10000
    d0, d1 = W.uniform_digraph()
    assert np.array_equal(c0, d0) and np.array_equal(c1, d1)


def test_rmat_graph_is_simple_and_skewed():
    c0, c1 = W.rmat_graph(12, 16)
    assert c0.max() < 4096 and c1.max() < 4096
    assert np.all(c0 != c1)
    k = W.pack_pairs(c0, c1)
    assert len(np.unique(k)) == len(k)
    deg = np.bincount(c0, minlength=4096)
    assert deg[0] > 20 * np.median(deg[deg > 0])      # a = 0.57 concentrates edges on low ids


def test_rmat_dag_climbs_bands():
    c0, c1 = W.rmat_dag(14, 8, bands=64)
    shift = 14 - 6
    assert np.all((c0 >> shift) < (c1 >> shift))       # every edge goes to a strictly higher band
    assert len(np.unique(W.pack_pairs(c0, c1))) == len(c0)


def test_tree_dag_config3_shape():
    c0, c1, level = W.tree_dag(5000, 0.05, 3)
    assert len(c0) == 4999 + 250
    assert np.all(c0 < c1)                              # parents and extra edges point forward
    kids = np.bincount(c0[:4999], minlength=5000)
    internal = kids[kids > 0]
    assert internal.max() <= 6 and np.sum(internal < 2) <= 1   # 2..6 children (the last parent may be cut short)
    assert level[0] == 0 and level.max() >= 5


def test_andersen_id_spaces():
    rel = W.andersen_program(0.001)
    V = 2000
    ao0, ao1 = rel["addressOf"]
    assert ao0.max() < V and ao1.min() >= V and ao1.max() < V + 1000
    for name in ("assign", "load", "store"):
        a, b = rel[name]
        assert a.max() < V and b.max() < V
        assert len(np.unique(W.pack_pairs(a, b))) == len(a)
    a, b = rel["assign"]
    assert np.all(a != b)
