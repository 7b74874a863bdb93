"""Group-by through the C ABI against the reference's known answers and the numpy restatement."""
import numpy as np
import pytest

from test_groupby_cpu import CASES, NP, case_inputs
from xlog_b200 import _abi as A
from xlog_b200.lib import XlbError

pytestmark = pytest.mark.gpu
CODE = {"u32": A.U32, "u64": A.U64}


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["cite"].split("/")[-1])
def test_groupby_kat(provider, case):
    cols, keys, aggs = case_inputs(case)
    buf = provider.create_buffer_from_slices(cols, [CODE[t] for t in case["types"]])
    out = provider.groupby_multi_agg(buf, keys, aggs)
    assert [c.tolist() for c in provider.download(out)] == case["expected"], case["cite"]
    want_types = [CODE[case["types"][k]] for k in keys] + [A.U64 if op in (A.AGG_COUNT, A.AGG_SUM) else CODE[case["types"][v]] for v, op in aggs]
    assert out.schema() == want_types


@pytest.mark.parametrize("rows,groups", [(1, 1), (9, 4), (5000, 37), (300_000, 1000), (1_000_003, 3)])
def test_groupby_random_against_numpy(provider, oracle, rows, groups):
    rng = np.random.default_rng(rows)
    k0 = rng.integers(0, groups, rows).astype(np.uint32)
    k1 = rng.integers(0, 2, rows).astype(np.uint64) << np.uint64(40)
    v32 = rng.integers(0, 2 ** 32, rows).astype(np.uint32)
    v64 = rng.integers(0, 2 ** 62, rows).astype(np.uint64)
    if rows > 100:
        k0[: rows // 2] = 0          # one group holds half the rows
    cols, types = [k0, k1, v32, v64], [A.U32, A.U64, A.U32, A.U64]
    aggs = [(2, A.AGG_SUM), (2, A.AGG_MIN), (2, A.AGG_MAX), (3, A.AGG_SUM), (3, A.AGG_MIN), (0, A.AGG_COUNT)]
    buf = provider.create_buffer_from_slices(cols, types)
    for keys in ([0], [1, 0]):
        got = provider.download(provider.groupby_multi_agg(buf, keys, aggs))
        want = oracle.groupby_columns(cols, keys, aggs)
        assert len(got) == len(want)
        for g, w in zip(got, want):
            assert g.dtype == w.dtype and np.array_equal(g, w)


def test_groupby_single_agg_and_symbol_keys(provider, oracle):
    k = np.array([7, 3, 7, 3, 9], np.uint32)
    v = np.array([1, 2, 3, 4, 5], np.uint32)
    buf = provider.create_buffer_from_slices([k, v], [A.SYMBOL, A.U32])
    out = provider.groupby_agg(buf, [0], A.AGG_MAX, 1)
    assert out.schema() == [A.SYMBOL, A.U32]
    assert [c.tolist() for c in provider.download(out)] == [[3, 7, 9], [4, 3, 5]]


def test_groupby_errors(provider):
    buf = provider.create_buffer_from_slices([np.array([1], np.uint32), np.array([2], np.int32)], [A.U32, A.I32])
    with pytest.raises(XlbError, match="at least one key column"):
        provider.groupby_multi_agg(buf, [], [(1, A.AGG_COUNT)])
    with pytest.raises(XlbError, match="at least one aggregation"):
        provider.groupby_multi_agg(buf, [0], [])
    with pytest.raises(XlbError, match=r"Key column 5 out of bounds \(arity 2\)"):
        provider.groupby_multi_agg(buf, [5], [(1, A.AGG_COUNT)])
    with pytest.raises(XlbError, match=r"Value column 2 out of bounds \(arity 2\)"):
        provider.groupby_multi_agg(buf, [0], [(2, A.AGG_COUNT)])
    with pytest.raises(XlbError, match="Sum currently requires U32 or U64 values") as e:
        provider.groupby_multi_agg(buf, [0], [(1, A.AGG_SUM)])
    assert e.value.status == A.ERR_TYPE
    with pytest.raises(XlbError, match="keys must be"):
        provider.groupby_multi_agg(buf, [1], [(0, A.AGG_COUNT)])
    # a count does not look at the value column's type
    assert [c.tolist() for c in provider.download(provider.groupby_multi_agg(buf, [0], [(1, A.AGG_COUNT)]))] == [[1], [1]]
