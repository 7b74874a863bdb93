"""The order-independent relation digest (host twin of ``xlb_rel_checksum``) without a GPU:
known answers of the 64-bit mixer, independence of row order, and the rule by which the digests of
disjoint shards combine into the digest of the whole relation."""
import numpy as np

from xlog_b200 import digest
from xlog_b200.dist import mix64

MASK = (1 << 64) - 1


def _fmix64(x: int) -> int:
    # the 64-bit finaliser of MurmurHash3, written out (public algorithm)
    x ^= x >> 33
    x = (x * 0xFF51AFD7ED558CCD) & MASK
    x ^= x >> 33
    x = (x * 0xC4CEB9FE1A85EC53) & MASK
    x ^= x >> 33
    return x


def test_mixer_matches_the_written_out_finaliser():
    xs = [0, 1, 2, 0xFFFFFFFF, 1 << 32, (5 << 32) | 7, MASK]
    got = mix64(np.array(xs, dtype=np.uint64))
    assert [int(g) for g in got] == [_fmix64(x) for x in xs]
    assert _fmix64(0) == 0 and _fmix64(1) == 0xB456BCFC34C2CB2C


def test_digest_is_count_xor_and_low_sum_of_the_mixed_rows():
    a = np.array([3, 1, 2], np.uint32)
    b = np.array([9, 8, 7], np.uint32)
    n, x, low = digest.result_checksum([a, b])
    mixed = [_fmix64((int(p) << 32) | int(q)) for p, q in zip(a, b)]
    assert n == 3 and x == mixed[0] ^ mixed[1] ^ mixed[2] and low == sum(m & 0xFFFFFFFF for m in mixed)
    # a one-column relation mixes the value itself
    n1, x1, low1 = digest.result_checksum([a])
    assert (n1, x1, low1) == (3, _fmix64(3) ^ _fmix64(1) ^ _fmix64(2), sum(_fmix64(v) & 0xFFFFFFFF for v in (3, 1, 2)))
    assert digest.result_checksum([]) == (0, 0, 0)
    assert digest.result_checksum([np.zeros(0, np.uint32), np.zeros(0, np.uint32)]) == (0, 0, 0)


def test_row_order_does_not_matter_and_shards_combine():
    rng = np.random.default_rng(5)
    a = rng.integers(0, 1 << 20, 100_000, dtype=np.uint32)
    b = rng.integers(0, 1 << 20, 100_000, dtype=np.uint32)
    whole = digest.result_checksum([a, b])
    perm = rng.permutation(len(a))
    assert digest.result_checksum([a[perm], b[perm]]) == whole
    cuts = [0, 10, 33_333, 70_001, len(a)]
    parts = [digest.result_checksum([a[lo:hi], b[lo:hi]]) for lo, hi in zip(cuts, cuts[1:])]
    assert digest.checksum_text(parts) == digest.checksum_text([whole])
    # one changed row changes the text
    b2 = b.copy()
    b2[17] ^= 1
    assert digest.checksum_text([digest.result_checksum([a, b2])]) != digest.checksum_text([whole])
