"""Order-independent digest of a relation's rows, the host-side twin of ``xlb_rel_checksum``.

``bench.py`` prints it so that the result of a fixpoint can be compared between rank counts and
with the CPU port; the device computes the same three numbers shard by shard.
"""
from __future__ import annotations

import numpy as np

from .dist import mix64


def result_checksum(cols) -> tuple[int, int, int]:
    """Order-independent digest of a set of tuples: (count, XOR, sum of the low 32 bits) of the
    64-bit mix of every packed tuple.  Shards of disjoint tuples combine by adding the counts and
    sums and XOR-ing the XORs, so the digest of a sharded result equals that of the whole."""
    n = len(cols[0]) if cols else 0
    if n == 0:
        return 0, 0, 0
    xor, low = 0, 0
    step = 1 << 24
    for at in range(0, n, step):
        k = cols[0][at:at + step].astype(np.uint64)
        if len(cols) > 1:
            k = (k << np.uint64(32)) | cols[1][at:at + step].astype(np.uint64)
        h = mix64(k)
        xor ^= int(np.bitwise_xor.reduce(h))
        low += int((h & np.uint64(0xFFFFFFFF)).sum(dtype=np.uint64))
    return n, xor, low


def checksum_text(parts) -> str:
    n = sum(p[0] for p in parts)
    xor = 0
    for p in parts:
        xor ^= p[1]
    low = sum(p[2] for p in parts) & ((1 << 64) - 1)
    return f"{n:x}-{xor:016x}-{low:016x}"
