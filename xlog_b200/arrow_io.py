"""Arrow IPC streams in and out of device relations: the wire format on either side of the path.

Mirrors ``CudaKernelProvider::{to,from}_arrow_ipc_stream`` and the ``*_file`` pair
(crates/xlog-cuda/src/provider/io.rs:345-773): one RecordBatch per stream, non-nullable fields,
column types Boolean / UInt32 / Int32 / UInt64 / Int64 / Float32 / Float64, and symbol columns as
``Dictionary<UInt32, Utf8>`` whose strings go through the symbol table
(crates/xlog-core/src/symbol.rs:30-131).  Not zero-copy: columns pass through host memory, as in
the reference.

The column functions need only pyarrow and numpy; the ``*_buffer`` functions add the upload and
download through a ``KernelProvider``.
"""
from __future__ import annotations

import threading
from typing import Sequence

import numpy as np
import pyarrow as pa

from . import _abi as A
from .lib import XlbError


class SymbolTable:
    """String <-> id registry: ids are handed out in order of first interning, starting at 0
    (symbol.rs:30-49).  One process-wide instance, ``SYMBOLS``, stands for the reference's global
    registry; tests may make their own."""

    def __init__(self):
        self._lock = threading.Lock()
        self._ids: dict[str, int] = {}
        self._strings: list[str] = []

    def intern(self, s: str) -> int:
        with self._lock:
            i = self._ids.get(s)
            if i is None:
                i = len(self._strings)
                self._ids[s] = i
                self._strings.append(s)
            return i

    def resolve(self, i: int) -> str:
        """The string of an id; ``KeyError`` for an id that was never handed out."""
        if 0 <= i < len(self._strings):
            return self._strings[i]
        raise KeyError(f"invalid symbol id {i}")

    def clear(self):
        with self._lock:
            self._ids.clear()
            self._strings.clear()

    def __len__(self):
        return len(self._strings)


SYMBOLS = SymbolTable()

_ARROW = {A.U32: pa.uint32(), A.U64: pa.uint64(), A.I32: pa.int32(), A.I64: pa.int64(),
          A.F32: pa.float32(), A.F64: pa.float64(), A.BOOL: pa.bool_()}
_NP = {A.U32: np.uint32, A.U64: np.uint64, A.I32: np.int32, A.I64: np.int64, A.F32: np.float32,
       A.F64: np.float64, A.BOOL: np.uint8, A.SYMBOL: np.uint32}
_SYMBOL_TYPE = pa.dictionary(pa.uint32(), pa.utf8())


def _symbol_array(ids: np.ndarray, symbols: SymbolTable) -> pa.DictionaryArray:
    # dictionary = the distinct ids in order of first appearance (symbol.rs:85-107)
    uniq, first, inverse = np.unique(ids, return_index=True, return_inverse=True)
    order = np.argsort(first, kind="stable")         # positions in `uniq`, by first appearance
    rank = np.empty(len(order), dtype=np.uint32)
    rank[order] = np.arange(len(order), dtype=np.uint32)
    keys = rank[inverse.reshape(-1)] if len(ids) else np.zeros(0, np.uint32)
    strings = pa.array([symbols.resolve(int(i)) for i in uniq[order]], type=pa.utf8())
    return pa.DictionaryArray.from_arrays(pa.array(keys, type=pa.uint32()), strings)


def columns_to_record_batch(cols: Sequence[np.ndarray], types: Sequence[int], names: Sequence[str] | None = None,
                            symbols: SymbolTable = SYMBOLS) -> pa.RecordBatch:
    if len(cols) != len(types):
        raise XlbError(A.ERR_INVALID, "one type per column")
    names = list(names) if names is not None else [f"c{i}" for i in range(len(cols))]
    if len(names) != len(cols):
        raise XlbError(A.ERR_INVALID, "one name per column")
    arrays, fields = [], []
    for c, t, n in zip(cols, types, names):
        c = np.ascontiguousarray(c, dtype=_NP[t])
        if t == A.SYMBOL:
            arrays.append(_symbol_array(c, symbols))
            fields.append(pa.field(n, _SYMBOL_TYPE, nullable=False))
        elif t == A.BOOL:
            arrays.append(pa.array(c != 0, type=pa.bool_()))
            fields.append(pa.field(n, pa.bool_(), nullable=False))
        else:
            arrays.append(pa.array(c, type=_ARROW[t]))
            fields.append(pa.field(n, _ARROW[t], nullable=False))
    return pa.record_batch(arrays, schema=pa.schema(fields))


def columns_to_ipc_stream(cols, types, names=None, symbols: SymbolTable = SYMBOLS) -> bytes:
    """Columns -> the bytes of an Arrow IPC stream holding one RecordBatch (io.rs:697-711)."""
    batch = columns_to_record_batch(cols, types, names, symbols)
    sink = pa.BufferOutputStream()
    with pa.ipc.new_stream(sink, batch.schema) as w:
        w.write_batch(batch)
    return sink.getvalue().to_pybytes()


def _type_of(dt: pa.DataType) -> int:
    for code, t in _ARROW.items():
        if dt == t:
            return code
    if pa.types.is_dictionary(dt) and dt.index_type == pa.uint32() and (pa.types.is_string(dt.value_type) or pa.types.is_large_string(dt.value_type)):
        return A.SYMBOL
    raise XlbError(A.ERR_TYPE, f"Unsupported Arrow type: {dt}")


def record_batch_to_columns(batch: pa.RecordBatch, symbols: SymbolTable = SYMBOLS):
    """-> (columns, type codes, names).  Nulls are not part of the format: a null value is an
    error (the reference maps a null boolean to false and panics on a null symbol; nothing
    writes them)."""
    cols, types, names = [], [], []
    for field, arr in zip(batch.schema, batch.columns):
        t = _type_of(field.type)
        if arr.null_count:
            raise XlbError(A.ERR_INVALID, f"column {field.name}: null values are not supported")
        if t == A.SYMBOL:
            ids = np.array([symbols.intern(s) for s in arr.dictionary.to_pylist()], dtype=np.uint32)
            keys = arr.indices.to_numpy(zero_copy_only=False).astype(np.int64)
            col = ids[keys] if len(keys) else np.zeros(0, np.uint32)
        elif t == A.BOOL:
            col = arr.to_numpy(zero_copy_only=False).astype(np.uint8)
        else:
            col = np.ascontiguousarray(arr.to_numpy(zero_copy_only=False), dtype=_NP[t])
        cols.append(col)
        types.append(t)
        names.append(field.name)
    return cols, types, names


def ipc_stream_to_columns(data: bytes, symbols: SymbolTable = SYMBOLS):
    """The one RecordBatch of an Arrow IPC stream -> (columns, type codes, names).  A stream with
    no batch or with more than one is an error, with the reference's messages (io.rs:722-739)."""
    try:
        reader = pa.ipc.open_stream(pa.BufferReader(data))
    except (pa.ArrowInvalid, OSError) as e:
        raise XlbError(A.ERR_INVALID, f"Failed to create Arrow IPC reader: {e}") from None
    try:
        batches = list(reader)
    except pa.ArrowInvalid as e:
        raise XlbError(A.ERR_INVALID, f"Failed to read Arrow RecordBatch: {e}") from None
    if not batches:
        raise XlbError(A.ERR_INVALID, "Arrow IPC stream contained no record batches")
    if len(batches) > 1:
        raise XlbError(A.ERR_INVALID, "Arrow IPC stream contains multiple record batches; this API expects exactly one")
    return record_batch_to_columns(batches[0], symbols)


# ---- with a provider -------------------------------------------------------------------------
def to_arrow_ipc_stream(provider, buf, names=None, symbols: SymbolTable = SYMBOLS) -> bytes:
    """Device relation -> Arrow IPC stream bytes (io.rs:697)."""
    return columns_to_ipc_stream(provider.download(buf), buf.schema(), names, symbols)


def from_arrow_ipc_stream(provider, data: bytes, symbols: SymbolTable = SYMBOLS):
    """Arrow IPC stream bytes -> device relation (io.rs:716).  Boolean columns are not a built
    column type of the library: they are refused with a type error."""
    cols, types, _ = ipc_stream_to_columns(data, symbols)
    if not cols or len(cols[0]) == 0:
        return provider.create_empty_buffer(types)
    return provider.create_buffer_from_slices(cols, types)


def write_arrow_ipc_stream_file(provider, buf, path, names=None, symbols: SymbolTable = SYMBOLS) -> None:
    data = to_arrow_ipc_stream(provider, buf, names, symbols)
    try:
        with open(path, "wb") as f:
            f.write(data)
    except OSError as e:
        raise XlbError(A.ERR_INVALID, f"Failed to write Arrow IPC stream to {path}: {e}") from None


def read_arrow_ipc_stream_file(provider, path, symbols: SymbolTable = SYMBOLS):
    try:
        with open(path, "rb") as f:
            data = f.read()
    except OSError as e:
        raise XlbError(A.ERR_INVALID, f"Failed to read Arrow IPC stream from {path}: {e}") from None
    return from_arrow_ipc_stream(provider, data, symbols)
