"""Group-by (groupby_multi_agg, crates/xlog-cuda/src/provider/groupby.rs:66): the numpy restatement
against the reference's known answers and against a dictionary-based count on random input."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = json.load(open(os.path.join(HERE, "golden", "groupby.json")))
OPS = {"count": 0, "sum": 1, "min": 2, "max": 3}
NP = {"u32": np.uint32, "u64": np.uint64}


def case_inputs(case):
    cols = [np.array(c, dtype=NP[t]) for c, t in zip(case["cols"], case["types"])]
    return cols, case["keys"], [(v, OPS[o]) for v, o in case["aggs"]]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["cite"].split("/")[-1])
def test_oracle_groupby_kat(oracle, case):
    cols, keys, aggs = case_inputs(case)
    out = oracle.groupby_columns(cols, keys, aggs)
    assert [c.tolist() for c in out] == case["expected"], case["cite"]
    for c, (v, op) in zip(out[len(keys):], aggs):
        assert c.dtype == (np.uint64 if op in (0, 1) else cols[v].dtype)   # groupby.rs:799-811


def test_oracle_groupby_against_a_dictionary(oracle):
    rng = np.random.default_rng(5)
    k0, k1 = rng.integers(0, 7, 500).astype(np.uint32), rng.integers(0, 3, 500).astype(np.uint64)
    v = rng.integers(0, 2 ** 40, 500).astype(np.uint64)
    want = {}
    for a, b, x in zip(k0.tolist(), k1.tolist(), v.tolist()):
        g = want.setdefault((a, b), [0, 0, 2 ** 64, 0])
        g[0] += 1
        g[1] += x
        g[2] = min(g[2], x)
        g[3] = max(g[3], x)
    out = oracle.groupby_columns([k0, k1, v], [0, 1], [(2, 0), (2, 1), (2, 2), (2, 3)])
    got = {(a, b): [c, s, lo, hi] for a, b, c, s, lo, hi in zip(*[c.tolist() for c in out])}
    assert got == want and list(got) == sorted(got)
