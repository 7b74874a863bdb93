"""A flat checkpoint of a fixpoint in progress: (full, delta, iteration), for resume.

One little-endian file:

    "XLBCKPT1"  u32 version (1)  u32 relations  u64 iteration
    per relation:  u32 name length, name (UTF-8, zero-padded to 8 bytes)
                   u32 arity, u8 types[8] (xlb_type codes), u32 flags (bit 0: sorted and unique)
                   u64 rows, then every column: rows * width bytes, zero-padded to 8 bytes
    u32 CRC-32 of everything before it, "XLBE"

The delta of a head relation travels under the name the executor keeps it by, ``__delta_<head>``.
A run that stops at the iteration limit with ``FLAG_KEEP_DELTAS`` leaves those in the store;
``save`` writes them with the full relations, ``restore`` puts everything back, and
``execute_plan`` then resumes every recursive SCC whose deltas it finds, without seeding it again.
The reference has no checkpoint: the file is this library's own.  With several ranks every rank
saves and restores its own shard, under the same rank count.
"""
from __future__ import annotations

import struct
import zlib
from typing import Iterable, Mapping, Sequence

import numpy as np

from . import _abi as A
from .lib import XlbError

MAGIC, END, VERSION = b"XLBCKPT1", b"XLBE", 1
_NP = {A.U32: np.uint32, A.U64: np.uint64, A.I32: np.int32, A.I64: np.int64, A.F32: np.float32, A.F64: np.float64,
       A.SYMBOL: np.uint32}


def _pad8(n: int) -> int:
    return (-n) % 8


def pack(relations: Mapping[str, tuple[Sequence[np.ndarray], Sequence[int], bool]], iteration: int) -> bytes:
    """``relations``: name -> (columns, type codes, sorted-and-unique flag)."""
    out = [MAGIC, struct.pack("<IIQ", VERSION, len(relations), iteration)]
    for name, (cols, types, canonical) in relations.items():
        nb = name.encode()
        if len(cols) != len(types) or len(types) > A.XLB_MAX_ARITY:
            raise XlbError(A.ERR_INVALID, f"checkpoint: relation {name!r} has {len(cols)} columns and {len(types)} types")
        rows = len(cols[0]) if cols else 0
        out += [struct.pack("<I", len(nb)), nb, b"\0" * _pad8(len(nb))]
        out.append(struct.pack("<I8sIQ", len(types), bytes(list(types) + [0] * (8 - len(types))), 1 if canonical else 0, rows))
        for c, t in zip(cols, types):
            if t not in _NP:
                raise XlbError(A.ERR_TYPE, f"checkpoint: column type {t} of {name!r} is not a built type")
            b = np.ascontiguousarray(c, dtype=_NP[t]).tobytes()
            if len(b) != rows * np.dtype(_NP[t]).itemsize:
                raise XlbError(A.ERR_INVALID, f"checkpoint: columns of {name!r} differ in length")
            out += [b, b"\0" * _pad8(len(b))]
    body = b"".join(out)
    return body + struct.pack("<I", zlib.crc32(body)) + END


def unpack(data: bytes):
    """-> (name -> (columns, type codes, flag), iteration).  Anything but a complete, unaltered
    file is an error."""
    def bad(what):
        raise XlbError(A.ERR_INVALID, f"checkpoint: {what}")

    if len(data) < len(MAGIC) + 16 + 8 or data[:8] != MAGIC:
        bad("not a checkpoint file")
    if data[-4:] != END:
        bad("the file is truncated")
    body, (crc,) = data[:-8], struct.unpack("<I", data[-8:-4])
    if zlib.crc32(body) != crc:
        bad("checksum mismatch")
    version, count, iteration = struct.unpack_from("<IIQ", body, 8)
    if version != VERSION:
        bad(f"version {version} is not supported")
    at, rels = 24, {}
    try:
        for _ in range(count):
            (nl,) = struct.unpack_from("<I", body, at)
            at += 4
            name = body[at:at + nl].decode()
            at += nl + _pad8(nl)
            arity, types, flags, rows = struct.unpack_from("<I8sIQ", body, at)
            at += struct.calcsize("<I8sIQ")
            if arity > A.XLB_MAX_ARITY:
                bad(f"relation {name!r}: arity {arity}")
            cols, tl = [], list(types[:arity])
            for t in tl:
                if t not in _NP:
                    bad(f"relation {name!r}: column type {t}")
                nbytes = rows * np.dtype(_NP[t]).itemsize
                if at + nbytes > len(body):
                    bad("the file is truncated")
                cols.append(np.frombuffer(body, dtype=_NP[t], count=rows, offset=at).copy())
                at += nbytes + _pad8(nbytes)
            rels[name] = (cols, tl, bool(flags & 1))
    except (struct.error, UnicodeDecodeError):
        bad("the file is truncated")
    if at != len(body):
        bad("trailing bytes")
    return rels, iteration


# ---- with an executor ------------------------------------------------------------------------
def save(executor, names: Iterable[str], path, iteration: int = 0) -> list[str]:
    """Write the named stored relations and, where the store holds it, the delta of each
    (``__delta_<name>``).  Returns the names written."""
    from .lib import XlbError as _E
    prov, rels = executor.provider, {}
    for base in names:
        for name in (base, "__delta_" + base):
            try:
                buf = executor.get(name)
            except _E as e:
                if name != base and e.status == A.ERR_NOT_FOUND:
                    continue
                raise
            rels[name] = (prov.download(buf), buf.schema(), buf.is_canonical())
    data = pack(rels, iteration)
    with open(path, "wb") as f:
        f.write(data)
    return list(rels)


def restore(executor, path) -> int:
    """Put every relation of the file into the executor's store; returns the iteration count.
    Relations come back as plain (uncertified) relations: the executor sorts and deduplicates what
    it needs, which leaves sorted unique rows as they are."""
    with open(path, "rb") as f:
        rels, iteration = unpack(f.read())
    prov = executor.provider
    for name, (cols, types, _) in rels.items():
        buf = prov.create_buffer_from_slices(cols, types) if cols and len(cols[0]) else prov.create_empty_buffer(types)
        executor.put_relation(name, buf)
    return iteration
