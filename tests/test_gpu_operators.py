"""The CUDA operators (through the C ABI) against the reference's known-answer fixtures, the CPU
oracle, and size-independent properties at tile boundaries."""
import numpy as np
import pytest

from test_oracle_golden import OPS, PROGS, cols_of, expected_of, rows_of, run_operator_case
from xlog_b200 import _abi as A
from xlog_b200.lib import XlbError

pytestmark = pytest.mark.gpu
T = {"u32": A.U32, "u64": A.U64, "i32": A.I32, "i64": A.I64, "f64": A.F64, "f32bits": A.F32}


class GpuOps:
    def __init__(self, p):
        self.p = p

    def make(self, rows, types):
        return self.p.create_buffer_from_slices(cols_of(rows, types), [T[t] for t in types])

    def rows(self, b):
        return rows_of(self.p.download(b))

    def sort(self, b, keys):
        return self.p.sort(b, keys)

    def dedup(self, b):
        return self.p.dedup_full_row(b)

    def union_many(self, bs):
        return self.p.union_many_gpu(bs)

    def diff(self, a, b):
        return self.p.diff_gpu(a, b)

    def hash_join(self, a, b, lk, rk, jt):
        return self.p.hash_join_v2(a, b, lk, rk, jt)


@pytest.mark.parametrize("case", [c for c in OPS if not c["op"].endswith("_error")], ids=lambda c: c["op"] + "@" + c["cite"].split(" ")[0])
def test_operator_kat(provider, case):
    ops = GpuOps(provider)
    got, want = expected_of(case, run_operator_case(case, ops.make, ops))
    assert got == want, case["cite"]


def test_union_errors(provider):
    ops = GpuOps(provider)
    with pytest.raises(XlbError) as e:
        provider.union_many_gpu([])
    assert e.value.status == A.ERR_INVALID
    with pytest.raises(XlbError) as e:
        provider.union_many_gpu([ops.make([[1]], ["u32"]), ops.make([[1, 2]], ["u32", "u32"])])
    assert e.value.status == A.ERR_TYPE
    with pytest.raises(XlbError) as e:
        provider.diff_gpu(ops.make([[1]], ["u32"]), ops.make([[1]], ["u64"]))
    assert e.value.status == A.ERR_TYPE
    with pytest.raises(XlbError) as e:
        provider.hash_join_v2(ops.make([[1]], ["u32"]), ops.make([[1]], ["u64"]), [0], [0])
    assert e.value.status == A.ERR_TYPE


def test_set_results_are_certified_and_inputs_untouched(provider):
    ops = GpuOps(provider)
    a = ops.make([[3, 1], [1, 2], [3, 1]], ["u32", "u32"])
    b = ops.make([[1, 2]], ["u32", "u32"])
    u = provider.union_gpu(a, b)
    d = provider.diff_gpu(a, b)
    assert u.is_canonical() and d.is_canonical() and not a.is_canonical()
    assert ops.rows(u) == [[1, 2], [3, 1]] and ops.rows(d) == [[3, 1]]
    assert ops.rows(a) == [[3, 1], [1, 2], [3, 1]]            # operators never mutate their inputs
    assert ops.rows(provider.clone_buffer(a)) == ops.rows(a)
    e = provider.create_empty_buffer([A.U32, A.U32])
    assert e.num_rows() == 0 and ops.rows(provider.union_gpu(e, e)) == []


def _keys(n, seed, bits):
    from xlog_b200.workloads import splitmix64
    return splitmix64(seed, 0, n) >> np.uint64(64 - bits)


SIZES = [1, 2, 31, 32, 33, 255, 256, 257, 2047, 2048, 2049, 4095, 4096, 4097, 8191, 8193, 100_003]


@pytest.mark.parametrize("n", SIZES)
def test_dedup_diff_union_against_numpy_at_tile_edges(provider, n):
    k = _keys(n, n, 18)             # 18-bit values: plenty of duplicates and overlaps
    m = _keys(max(n // 2, 1), n + 7, 18)
    ka = [(k >> np.uint64(9)).astype(np.uint32), (k & np.uint64(511)).astype(np.uint32)]
    kb = [(m >> np.uint64(9)).astype(np.uint32), (m & np.uint64(511)).astype(np.uint32)]
    a = provider.create_buffer_from_slices(ka)
    b = provider.create_buffer_from_slices(kb)
    pa = (ka[0].astype(np.uint64) << np.uint64(32)) | ka[1]
    pb = (kb[0].astype(np.uint64) << np.uint64(32)) | kb[1]

    def packed(buf):
        c = provider.download(buf)
        return (c[0].astype(np.uint64) << np.uint64(32)) | c[1]

    assert np.array_equal(packed(provider.dedup(a)), np.unique(pa))
    assert np.array_equal(packed(provider.diff_gpu(a, b)), np.setdiff1d(pa, pb))
    assert np.array_equal(packed(provider.union_gpu(a, b)), np.union1d(pa, pb))
    da = provider.dedup(a)
    assert np.array_equal(packed(provider.dedup(da)), packed(da))                 # idempotent
    assert provider.diff_gpu(a, a).num_rows() == 0                                # a \ a is empty
    assert np.array_equal(packed(provider.union_gpu(da, da)), packed(da))         # a U a = a
    s = provider.download(provider.sort(a, [1, 0]))                               # stable two-key sort
    order = np.lexsort((ka[0], ka[1]))
    assert np.array_equal(s[0], ka[0][order]) and np.array_equal(s[1], ka[1][order])


@pytest.mark.parametrize("n", [1, 33, 2049, 50_000])
def test_stable_sort_carries_payload_columns(provider, n):
    k = _keys(n, 3, 6).astype(np.uint32)                      # few distinct keys: stability is visible
    pay = np.arange(n, dtype=np.uint32)
    wide = _keys(n, 4, 40)
    out = provider.download(provider.sort(provider.create_buffer_from_slices([k, pay, wide], [A.U32, A.U32, A.U64]), [0]))
    order = np.argsort(k, kind="stable")
    assert np.array_equal(out[0], k[order]) and np.array_equal(out[1], pay[order]) and np.array_equal(out[2], wide[order])


@pytest.mark.parametrize("nl,nr,bits", [(1, 1, 2), (1000, 37, 5), (5000, 5000, 10), (40_000, 3000, 8)])
def test_inner_semi_anti_join_against_oracle(provider, oracle, nl, nr, bits):
    l = [_keys(nl, 1, bits).astype(np.uint32), np.arange(nl, dtype=np.uint32)]
    r = [_keys(nr, 2, bits).astype(np.uint32), np.arange(nr, dtype=np.uint32) + 7]
    gl, gr = provider.create_buffer_from_slices(l), provider.create_buffer_from_slices(r)
    ol, orr = oracle.OracleRel.from_columns(l), oracle.OracleRel.from_columns(r)
    for jt in (A.JOIN_INNER, A.JOIN_SEMI, A.JOIN_ANTI):
        got = provider.download(provider.hash_join_v2(gl, gr, [0], [0], jt))
        want = oracle.hash_join(ol, orr, [0], [0], jt).columns()
        # the inner join is ordered by left row then right row on both sides: compare as is
        assert len(got) == len(want)
        for g, w in zip(got, want):
            assert np.array_equal(g, w)


def test_wide_rows_and_u64_columns(provider, oracle):
    n = 3000
    cols = [_keys(n, 1, 3), _keys(n, 2, 3), _keys(n, 3, 2)]
    other = [_keys(500, 4, 3), _keys(500, 5, 3), _keys(500, 6, 2)]
    a = provider.create_buffer_from_slices(cols, [A.U64] * 3)
    b = provider.create_buffer_from_slices(other, [A.U64] * 3)
    oa = oracle.OracleRel.from_columns(cols, dtype=np.uint64)
    ob = oracle.OracleRel.from_columns(other, dtype=np.uint64)
    for got, want in ((provider.dedup(a), oracle.dedup(oa)), (provider.union_gpu(a, b), oracle.union_many([oa, ob])),
                      (provider.diff_gpu(a, b), oracle.diff(oa, ob))):
        assert got.is_canonical()
        for g, w in zip(provider.download(got), want.columns()):
            assert np.array_equal(g, w)


def test_partial_key_dedup_keeps_first_row_per_key(provider, oracle):
    k = _keys(5000, 8, 7).astype(np.uint32)
    pay = np.arange(5000, dtype=np.uint32)
    got = provider.download(provider.dedup(provider.create_buffer_from_slices([k, pay]), [0]))
    want = oracle.dedup(oracle.OracleRel.from_columns([k, pay]), [0]).columns()
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_zero_arity_relations(provider):
    empty = provider.create_buffer_from_slices([], [])
    assert empty.num_rows() == 0 and provider.union_many_gpu([empty]).num_rows() == 0
    assert provider.diff_gpu(empty, empty).num_rows() == 0


def test_same_input_twice_gives_identical_bytes(provider):
    k = _keys(200_000, 21, 30)
    cols = [(k >> np.uint64(15)).astype(np.uint32), (k & np.uint64(32767)).astype(np.uint32)]
    a = provider.create_buffer_from_slices(cols)
    r1 = provider.download(provider.hash_join_v2(provider.dedup(a), a, [1], [0]))
    r2 = provider.download(provider.hash_join_v2(provider.dedup(a), a, [1], [0]))
    assert all(x.tobytes() == y.tobytes() for x, y in zip(r1, r2))


def test_memory_budget_is_enforced():
    from xlog_b200.provider import KernelProvider
    p = KernelProvider(device=0, memory_budget_bytes=1 << 20)
    big = np.zeros(1 << 20, dtype=np.uint32)
    with pytest.raises(XlbError) as e:
        p.create_buffer_from_slices([big, big])
    assert e.value.status == A.ERR_RESOURCE_EXHAUSTED and "budget" in e.value.message
    small = p.create_buffer_from_slices([big[:1000], big[:1000]])      # the context stays usable
    assert p.dedup(small).num_rows() == 1
    p.close()


def test_typed_columns_against_oracle(provider, oracle):
    """Signed and floating columns: the reference's typed order (sign flip, IEEE totalOrder) and
    bitwise equality, on random data with negative values, infinities, NaNs and signed zeros."""
    n = 20_000
    raw = _keys(n, 31, 32).astype(np.uint32)
    i32 = (raw % np.uint32(401)).astype(np.int64) - 200
    f32 = ((raw >> np.uint32(9)) % np.uint32(64)).astype(np.float32) - np.float32(32.0)
    f32[::97] = np.float32("nan")
    f32[1::97] = np.float32("-inf")
    f32[2::97] = np.float32(-0.0)
    cols = [i32.astype(np.int32), f32]
    other = [cols[0][::3].copy(), cols[1][::3].copy()]
    a = provider.create_buffer_from_slices(cols)
    b = provider.create_buffer_from_slices(other)
    assert a.schema() == [A.I32, A.F32]
    oa, ob = oracle.OracleRel.from_columns(cols), oracle.OracleRel.from_columns(other)
    pairs = [(provider.dedup(a), oracle.dedup(oa)), (provider.diff_gpu(a, b), oracle.diff(oa, ob)),
             (provider.union_gpu(a, b), oracle.union_many([oa, ob])), (provider.sort(a, [1, 0]), oracle.sort(oa, [1, 0]))]
    for got, want in pairs:
        assert got.schema() == [A.I32, A.F32]
        for g, w in zip(provider.download(got), want.columns()):
            assert g.dtype == w.dtype and g.tobytes() == w.tobytes()
    i64 = (_keys(n, 5, 40).astype(np.int64) - (1 << 39))
    f64 = i64.astype(np.float64) * 0.5
    got = provider.download(provider.dedup(provider.create_buffer_from_slices([i64, f64])))
    order = np.lexsort((f64, i64))
    assert np.array_equal(got[0], i64[order]) and np.array_equal(got[1], f64[order])      # all rows distinct here
    with pytest.raises(XlbError) as e:
        provider.union_gpu(provider.create_buffer_from_slices([i32.astype(np.int32)]),
                           provider.create_buffer_from_slices([raw]))
    assert e.value.status == A.ERR_TYPE


@pytest.mark.parametrize("nl", [2048, 2049, 8192, 8193, 2_097_152, 2_097_153])
def test_join_at_the_size_edges_of_the_prefix_sum(provider, nl):
    # the join scans one match length per left row: a single tile up to 2048 entries, one block up
    # to 8192, two launches up to 1024 tiles (2 097 152 entries), three beyond
    lk = (np.arange(nl, dtype=np.uint64) * np.uint64(2654435761) % np.uint64(1000)).astype(np.uint32)
    l = [lk, np.arange(nl, dtype=np.uint32)]
    r = [np.arange(0, 1000, 2, dtype=np.uint32), np.arange(0, 1000, 2, dtype=np.uint32) + 5]   # even keys only, once each
    out = provider.download(provider.hash_join_v2(provider.create_buffer_from_slices(l), provider.create_buffer_from_slices(r), [0], [0]))
    keep = lk % 2 == 0
    assert np.array_equal(out[0], lk[keep]) and np.array_equal(out[1], l[1][keep])     # left row order kept
    assert np.array_equal(out[2], lk[keep]) and np.array_equal(out[3], lk[keep] + 5)


def test_device_checksum_matches_the_host_digest_and_combines_over_shards(provider):
    """xlb_rel_checksum: the digest bench.py compares across rank counts.  The device result must
    equal the same function computed with numpy, and digests of disjoint shards must combine to the
    digest of the whole (also for rows of three columns, which are folded column by column)."""
    from xlog_b200.digest import checksum_text, result_checksum
    from xlog_b200.dist import mix64
    from xlog_b200.workloads import splitmix64
    n = 100_003
    c0 = (splitmix64(3, 0, n) >> np.uint64(40)).astype(np.uint32)
    c1 = (splitmix64(4, 0, n) >> np.uint64(38)).astype(np.uint32)
    whole = provider.checksum(provider.create_buffer_from_slices([c0, c1]))
    assert checksum_text([whole]) == checksum_text([result_checksum([c0, c1])])
    cut = 40_000
    parts = [provider.checksum(provider.create_buffer_from_slices([c0[:cut], c1[:cut]])),
             provider.checksum(provider.create_buffer_from_slices([c0[cut:], c1[cut:]]))]
    assert checksum_text(parts) == checksum_text([whole])
    one = provider.checksum(provider.create_buffer_from_slices([c0]))
    assert checksum_text([one]) == checksum_text([result_checksum([c0])])
    # three columns: h = mix(mix(mix(0 ^ a) ^ b) ^ c), mixed once more
    c2 = (splitmix64(5, 0, n) >> np.uint64(50)).astype(np.uint32)
    h = np.zeros(n, np.uint64)
    for col in (c0, c1, c2):
        h = mix64(h ^ col.astype(np.uint64))
    h = mix64(h)
    want = (n, int(np.bitwise_xor.reduce(h)), int((h & np.uint64(0xFFFFFFFF)).sum(dtype=np.uint64)))
    assert provider.checksum(provider.create_buffer_from_slices([c0, c1, c2])) == want
