"""The CPU oracle against independent numpy / pure-Python restatements on random relations: a
second pin beside the reference's known answers, for sizes and types those do not reach."""
import numpy as np
import pytest


def _rel(rng, rows, arity, hi, dtype=np.uint32):
    return [rng.integers(0, hi, rows).astype(dtype) for _ in range(arity)]


def _tuples(cols):
    return list(zip(*[c.tolist() for c in cols])) if cols and len(cols[0]) else []


@pytest.mark.parametrize("rows,arity,hi,dtype", [(0, 2, 5, np.uint32), (1, 1, 5, np.uint32), (500, 2, 12, np.uint32),
                                                  (3000, 3, 6, np.uint32), (800, 2, 9, np.uint64), (700, 4, 3, np.uint64)])
def test_set_operators(oracle, rows, arity, hi, dtype):
    rng = np.random.default_rng(rows * 7 + arity)
    a, b = _rel(rng, rows, arity, hi, dtype), _rel(rng, max(rows // 2, 0), arity, hi, dtype)
    ra, rb = oracle.OracleRel.from_columns(a, arity=arity), oracle.OracleRel.from_columns(b, arity=arity)
    sa, sb = set(_tuples(a)), set(_tuples(b))
    d = oracle.dedup(ra)
    assert d.tuples() == sorted(sa) and d.canonical
    assert oracle.union_many([ra, rb]).tuples() == sorted(sa | sb)
    assert oracle.diff(ra, rb).tuples() == sorted(sa - sb)
    assert oracle.diff(ra, ra).tuples() == []
    assert oracle.union_many([ra]).tuples() == sorted(sa)


@pytest.mark.parametrize("keys", [[0], [1, 0], [2], [0, 1, 2]])
def test_sort_is_stable_and_lexicographic(oracle, keys):
    rng = np.random.default_rng(len(keys))
    cols = _rel(rng, 2000, 3, 7)
    got = oracle.sort(oracle.OracleRel.from_columns(cols), keys).columns()
    order = np.lexsort([cols[k] for k in reversed(keys)])          # stable, first key most significant
    for g, c in zip(got, cols):
        assert np.array_equal(g, c[order])


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
def test_typed_order(oracle, dtype):
    rng = np.random.default_rng(3)
    if np.dtype(dtype).kind == "i":
        info = np.iinfo(dtype)
        v = np.concatenate([rng.integers(-50, 50, 300), [info.min, info.max, 0, -1]]).astype(dtype)
    else:
        v = np.concatenate([rng.normal(0, 10, 300), [np.inf, -np.inf, 0.0, -0.0, 1e-30, -1e-30]]).astype(dtype)
    got = oracle.sort(oracle.OracleRel.from_columns([v]), [0]).columns()[0]
    assert got.dtype == np.dtype(dtype)
    if np.dtype(dtype).kind == "i":
        assert np.array_equal(got, np.sort(v, kind="stable"))
    else:
        # IEEE totalOrder: as numeric order, with -0.0 before +0.0
        assert np.all(got[:-1] <= got[1:]) and sorted(got.tolist()) == sorted(v.tolist())
        zeros = got[got == 0]
        assert list(np.signbit(zeros)) == sorted(np.signbit(zeros), reverse=True)
    uniq = oracle.dedup(oracle.OracleRel.from_columns([v])).columns()[0]
    bits = v.view(np.uint32 if np.dtype(dtype).itemsize == 4 else np.uint64)
    assert len(uniq) == len(np.unique(bits))                       # equality is bitwise: -0.0 and +0.0 differ


def test_nan_sorts_by_sign_at_the_ends(oracle):
    # totalOrder: -NaN < -inf < ... < +inf < +NaN (kernels/totalorder.cuh)
    v = np.array([1.0, np.nan, -np.inf, np.copysign(np.nan, -1.0), np.inf, 0.0], dtype=np.float64)
    assert np.signbit(v[3]) and not np.signbit(v[1])
    got = oracle.sort(oracle.OracleRel.from_columns([v]), [0]).columns()[0]
    assert np.isnan(got[0]) and np.signbit(got[0]) and got[1] == -np.inf
    assert np.isnan(got[-1]) and not np.signbit(got[-1]) and got[-2] == np.inf
    assert got[2:4].tolist() == [0.0, 1.0]


@pytest.mark.parametrize("jt", [0, 1, 2])
def test_join_against_a_dictionary(oracle, jt):
    rng = np.random.default_rng(jt)
    l, r = _rel(rng, 400, 2, 20), _rel(rng, 150, 2, 20)
    got = oracle.hash_join(oracle.OracleRel.from_columns(l), oracle.OracleRel.from_columns(r), [0], [1], jt).tuples()
    by_key = {}
    for t in _tuples(r):
        by_key.setdefault(t[1], []).append(t)
    if jt == 0:      # every left row with every right row of its key (bag: duplicates kept)
        want = [lt + rt for lt in _tuples(l) for rt in by_key.get(lt[0], [])]
        assert sorted(got) == sorted(want) and len(got) == len(want)
    elif jt == 1:    # left rows with a partner, once each, left order kept
        assert got == [lt for lt in _tuples(l) if lt[0] in by_key]
    else:
        assert got == [lt for lt in _tuples(l) if lt[0] not in by_key]


@pytest.mark.parametrize("nodes,edges,seed", [(12, 20, 1), (60, 150, 2), (200, 380, 3)])
def test_fixpoints_against_boolean_matrix_closure(oracle, nodes, edges, seed):
    from xlog_b200 import programs
    rng = np.random.default_rng(seed)
    c0, c1 = rng.integers(0, nodes, edges).astype(np.uint32), rng.integers(0, nodes, edges).astype(np.uint32)
    adj = np.zeros((nodes, nodes), dtype=bool)
    adj[c0, c1] = True
    reach = adj.copy()
    while True:                                   # paths of length >= 1, by repeated squaring-free closure
        nxt = reach | (reach.astype(np.uint8) @ adj.astype(np.uint8) > 0)
        if np.array_equal(nxt, reach):
            break
        reach = nxt
    xs, ys = np.nonzero(reach)
    out, _ = oracle.run_program(programs.transitive_closure(), {"edge": [c0, c1]}, ["reach"])
    assert np.array_equal(out["reach"][0], xs.astype(np.uint32)) and np.array_equal(out["reach"][1], ys.astype(np.uint32))
    for builder in (programs.transitive_closure_left_linear, programs.transitive_closure_nonlinear):
        alt, _ = oracle.run_program(builder(), {"edge": [c0, c1]}, ["reach"])
        assert all(np.array_equal(a, b) for a, b in zip(alt["reach"], out["reach"]))
    src = int(c0[0])
    r, _ = oracle.run_program(programs.reach_from_source(src), {"edge": [c0, c1]}, ["r"])
    assert np.array_equal(r["r"][0], np.nonzero(reach[src])[0].astype(np.uint32))
