"""The checkpoint file format without a GPU: round trip, and every kind of damage is refused."""
import struct

import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import checkpoint as CK
from xlog_b200.lib import XlbError


def _rels():
    return {"reach": ([np.array([1, 1, 2], np.uint32), np.array([2, 3, 3], np.uint32)], [A.U32, A.U32], True),
            "__delta_reach": ([np.array([1], np.uint32), np.array([3], np.uint32)], [A.U32, A.U32], True),
            "w": ([np.array([5, 6, 7], np.uint64), np.array([-1, 0, 1], np.int32), np.array([0.5, 1.5, -2.0], np.float64)],
                  [A.U64, A.I32, A.F64], False),
            "empty": ([np.zeros(0, np.uint32)], [A.SYMBOL], False)}


def test_round_trip():
    data = CK.pack(_rels(), 17)
    assert len(data) % 4 == 0 and data[:8] == b"XLBCKPT1" and data[-4:] == b"XLBE"
    rels, it = CK.unpack(data)
    assert it == 17 and list(rels) == list(_rels())
    for name, (cols, types, flag) in _rels().items():
        gc, gt, gf = rels[name]
        assert gt == list(types) and gf == flag and len(gc) == len(cols)
        for g, c in zip(gc, cols):
            assert g.dtype == c.dtype and np.array_equal(g, c)


def test_damage_is_refused():
    data = CK.pack(_rels(), 3)
    with pytest.raises(XlbError, match="not a checkpoint"):
        CK.unpack(b"XLBCKPT0" + data[8:])
    with pytest.raises(XlbError, match="truncated"):
        CK.unpack(data[:-5])
    flipped = bytearray(data)
    flipped[40] ^= 1
    with pytest.raises(XlbError, match="checksum"):
        CK.unpack(bytes(flipped))
    # a well-formed file of another version
    body = b"XLBCKPT1" + struct.pack("<IIQ", 2, 0, 0)
    import zlib
    with pytest.raises(XlbError, match="version 2"):
        CK.unpack(body + struct.pack("<I", zlib.crc32(body)) + b"XLBE")
    with pytest.raises(XlbError, match="not a checkpoint"):
        CK.unpack(b"")


def test_malformed_relations_are_refused_when_writing():
    with pytest.raises(XlbError, match="differ in length"):
        CK.pack({"r": ([np.zeros(2, np.uint32), np.zeros(3, np.uint32)], [A.U32, A.U32], False)}, 0)
    with pytest.raises(XlbError, match="not a built type"):
        CK.pack({"r": ([np.zeros(2, np.uint8)], [A.BOOL], False)}, 0)
