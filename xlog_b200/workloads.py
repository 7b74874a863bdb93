"""Seeded synthetic inputs for the five benchmark configurations.

Every generator is a pure function of (parameters, seed) built on a counter-based
SplitMix64 stream, so the CPU oracle, the CUDA path and any other consumer read
bit-identical edge lists on any machine.  All relations are returned as
column-major ``numpy.uint32`` arrays, one array per column, the layout the
reference keeps on the device (crates/xlog-cuda/src/memory.rs:1758-1774).

No item of any public benchmark suite is reproduced here: "R-MAT" names only the
recursive-quadrant edge distribution with the stated (a, b, c, d).
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64(seed: int, start: int, count: int) -> np.ndarray:
    """``count`` outputs of SplitMix64 for counters ``start .. start+count-1``.

    Output i is ``mix(seed + (i+1) * golden)``, i.e. the i-th value of the
    sequential generator seeded with ``seed``, so any slice can be produced
    independently (and in parallel) of the others.
    """
    with np.errstate(over="ignore"):
        idx = np.arange(start + 1, start + count + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + idx * _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        z = z ^ (z >> np.uint64(31))
    return z


def config_seed(config: int) -> int:
    """Per-configuration seed: the SplitMix64 constant xor the config number."""
    return 0x9E3779B97F4A7C15 ^ int(config)


def _uniform_below(seed: int, start: int, count: int, n: int) -> np.ndarray:
    """``count`` integers in [0, n) (multiply-shift on the top 32 bits; n < 2**32)."""
    r = splitmix64(seed, start, count) >> np.uint64(32)
    return ((r * np.uint64(n)) >> np.uint64(32)).astype(np.uint32)


def pack_pairs(c0: np.ndarray, c1: np.ndarray) -> np.ndarray:
    """(c0 << 32) | c1 as uint64: ascending order == lexicographic (c0, c1)."""
    return (c0.astype(np.uint64) << np.uint64(32)) | c1.astype(np.uint64)


def unpack_pairs(k: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    return (k >> np.uint64(32)).astype(np.uint32), (k & np.uint64(0xFFFFFFFF)).astype(np.uint32)


def _dedup_pairs(c0, c1, drop_loops=True):
    if drop_loops:
        keep = c0 != c1
        c0, c1 = c0[keep], c1[keep]
    k = np.unique(pack_pairs(c0, c1))
    return unpack_pairs(k)


# --------------------------------------------------------------------------- C1
def uniform_digraph(nodes: int = 2000, edges: int = 10000, seed: int | None = None):
    """Config 1: ``edges`` distinct (u, v), u != v, uniform over ``nodes`` ids.

    Draws in rounds until enough distinct pairs exist, then keeps the first
    ``edges`` in draw order (so the relation is *not* sorted on arrival).
    """
    seed = config_seed(1) if seed is None else seed
    seen: dict[int, None] = {}
    pos = 0
    while len(seen) < edges:
        n = max(1024, 2 * (edges - len(seen)))
        u = _uniform_below(seed, pos, n, nodes)
        v = _uniform_below(seed ^ 0x5555555555555555, pos, n, nodes)
        pos += n
        for a, b in zip(u.tolist(), v.tolist()):
            if a != b and (a, b) not in seen:
                seen[(a, b)] = None
                if len(seen) == edges:
                    break
    arr = np.array(list(seen.keys()), dtype=np.uint32).reshape(-1, 2)
    return np.ascontiguousarray(arr[:, 0]), np.ascontiguousarray(arr[:, 1])


# ---------------------------------------------------------------------- R-MAT
def rmat_edges(scale: int, edge_factor: int, seed: int, a=0.57, b=0.19, c=0.19,
               chunk: int = 1 << 22):
    """Raw R-MAT edge list: ``edge_factor << scale`` (src, dst) pairs, ids < 2**scale.

    One 16-bit uniform per bit level picks the quadrant: [0,a) -> (0,0),
    [a,a+b) -> (0,1), [a+b,a+b+c) -> (1,0), rest -> (1,1); probabilities are
    therefore quantised to 1/65536.  Four levels are drawn from one SplitMix64
    word.  No vertex permutation is applied.
    """
    m = edge_factor << scale
    ta, tb, tc = (int(round(x * 65536)) for x in (a, a + b, a + b + c))
    words = (scale + 3) // 4
    src = np.empty(m, dtype=np.uint32)
    dst = np.empty(m, dtype=np.uint32)
    for lo in range(0, m, chunk):
        n = min(chunk, m - lo)
        s = np.zeros(n, dtype=np.uint32)
        d = np.zeros(n, dtype=np.uint32)
        level = 0
        for w in range(words):
            r = splitmix64(seed + 0x1000003 * w, lo, n)
            for q in range(4):
                if level == scale:
                    break
                x = ((r >> np.uint64(16 * q)) & np.uint64(0xFFFF)).astype(np.uint32)
                sbit = (x >= tb).astype(np.uint32)
                dbit = (((x >= ta) & (x < tb)) | (x >= tc)).astype(np.uint32)
                s = (s << np.uint32(1)) | sbit
                d = (d << np.uint32(1)) | dbit
                level += 1
        src[lo:lo + n] = s
        dst[lo:lo + n] = d
    return src, dst


def shuffle_rows(cols, seed: int):
    """The same rows in a seeded pseudo-random order (deduplication leaves them sorted; a
    consumer must not be handed that order for free)."""
    perm = np.argsort(splitmix64(seed ^ 0x0DDC0FFEE, 0, len(cols[0])), kind="stable")
    return tuple(np.ascontiguousarray(c[perm]) for c in cols)


def rmat_graph(scale: int = 20, edge_factor: int = 16, seed: int | None = None, shuffle: bool = True):
    """Config 2 input: R-MAT (a=.57 b=.19 c=.19 d=.05), self-loops and duplicates removed,
    rows in a seeded pseudo-random order (``shuffle=False`` keeps the (src, dst) order that
    deduplication leaves)."""
    seed = config_seed(2) if seed is None else seed
    s, d = rmat_edges(scale, edge_factor, seed)
    out = _dedup_pairs(s, d)
    return shuffle_rows(out, seed) if shuffle else out


def rmat_dag(scale: int = 24, edge_factor: int = 8, bands: int = 64, seed: int | None = None):
    """Config 5 input: R-MAT oriented low id -> high id, restricted to ``bands`` id-bands.

    The id space [0, 2**scale) is cut into ``bands`` equal contiguous bands.  An
    edge is kept only if, after orienting it low -> high, it goes to a strictly
    higher band.  Every path therefore climbs at least one band per hop, so the
    graph is acyclic and no path has more than ``bands - 1`` edges: the fixpoint
    needs at most ``bands`` iterations.  Duplicates are removed.
    """
    seed = config_seed(5) if seed is None else seed
    s, d = rmat_edges(scale, edge_factor, seed)
    lo = np.minimum(s, d)
    hi = np.maximum(s, d)
    shift = np.uint32(max(scale - int(np.log2(bands)), 0))
    keep = (lo >> shift) < (hi >> shift)
    return _dedup_pairs(lo[keep], hi[keep], drop_loops=False)


# --------------------------------------------------------------------------- C3
def tree_dag(nodes: int = 200_000, extra_frac: float = 0.05, seed: int | None = None):
    """Config 3 input: random tree (2-6 children per internal node, BFS order) plus
    ``extra_frac * nodes`` extra forward edges (low id -> higher id, not already present).

    edge(P, C): column 0 is the parent.  Returns (c0, c1, level_of_node).
    """
    seed = config_seed(3) if seed is None else seed
    fan = _uniform_below(seed, 0, nodes, 5).astype(np.int64) + 2      # uniform 2..6
    parent = np.zeros(nodes, dtype=np.uint32)
    level = np.zeros(nodes, dtype=np.uint32)
    nxt = 1
    p = 0
    while nxt < nodes:
        k = int(min(fan[p], nodes - nxt))
        parent[nxt:nxt + k] = p
        level[nxt:nxt + k] = level[p] + 1
        nxt += k
        p += 1
    c0 = parent[1:].copy()
    c1 = np.arange(1, nodes, dtype=np.uint32)
    n_extra = int(round(extra_frac * nodes))
    have = set(pack_pairs(c0, c1).tolist())
    ex0, ex1 = [], []
    pos = 0
    while len(ex0) < n_extra:
        n = 2 * (n_extra - len(ex0)) + 16
        u = _uniform_below(seed ^ 0xA5A5A5A5, pos, n, nodes)
        v = _uniform_below(seed ^ 0x5A5A5A5A, pos, n, nodes)
        pos += n
        for x, y in zip(u.tolist(), v.tolist()):
            if x == y:
                continue
            lo_, hi_ = (x, y) if x < y else (y, x)
            key = (lo_ << 32) | hi_
            if key in have:
                continue
            have.add(key)
            ex0.append(lo_)
            ex1.append(hi_)
            if len(ex0) == n_extra:
                break
    c0 = np.concatenate([c0, np.array(ex0, dtype=np.uint32)])
    c1 = np.concatenate([c1, np.array(ex1, dtype=np.uint32)])
    return c0, c1, level


# --------------------------------------------------------------------------- C4
def _zipf_below(seed: int, start: int, count: int, n: int, s: float = 1.1) -> np.ndarray:
    """``count`` ranks in [0, n) with P(rank r) ~ (r+1)**-s, by inverting the
    continuous power-law CDF (exact Zipf is not needed, only its skew)."""
    u = (splitmix64(seed, start, count) >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    one_minus_s = 1.0 - s
    hi = float(n + 1) ** one_minus_s
    x = (1.0 + u * (hi - 1.0)) ** (1.0 / one_minus_s)
    r = np.floor(x).astype(np.int64) - 1
    return np.clip(r, 0, n - 1).astype(np.uint32)


def andersen_program(scale: float = 1.0, seed: int | None = None):
    """Config 4 input: four relations of (u32, u32) facts for an Andersen-style analysis.

    ids: variables 0 .. V-1, heap objects V .. V+H-1 (one id space, so an object can
    sit in column 0 of pointsTo).  At scale 1: V = 2 M, H = 1 M, 4 M assign, 1 M
    load, 1 M store, 1 M addressOf draws; variable popularity is Zipf(1.1) over a
    fixed pseudo-random permutation of the variable ids; duplicates are removed.

    Returns dict name -> (c0, c1):
      addressOf(V, O), assign(V, W) [V = W], load(V, P) [V = *P], store(P, V) [*P = V].
    """
    seed = config_seed(4) if seed is None else seed
    V = max(int(2_000_000 * scale), 16)
    H = max(int(1_000_000 * scale), 8)
    n_assign = max(int(4_000_000 * scale), 8)
    n_other = max(int(1_000_000 * scale), 4)
    perm_keys = splitmix64(seed ^ 0x7777, 0, V)
    perm = np.argsort(perm_keys, kind="stable").astype(np.uint32)

    def zvars(tag, n):
        return perm[_zipf_below(seed ^ tag, 0, n, V)]

    out = {}
    out["addressOf"] = _dedup_pairs(zvars(0x11, n_other),
                                    _uniform_below(seed ^ 0x12, 0, n_other, H) + np.uint32(V),
                                    drop_loops=False)
    out["assign"] = _dedup_pairs(zvars(0x21, n_assign), zvars(0x22, n_assign))
    out["load"] = _dedup_pairs(zvars(0x31, n_other), zvars(0x32, n_other), drop_loops=False)
    out["store"] = _dedup_pairs(zvars(0x41, n_other), zvars(0x42, n_other), drop_loops=False)
    return out
