"""Arrow IPC stream format of relations (crates/xlog-cuda/src/provider/io.rs:345-773) without a
GPU: the column <-> stream functions, checked against pyarrow's own reader and writer."""
import numpy as np
import pyarrow as pa
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import arrow_io as AIO
from xlog_b200.lib import XlbError


def _stream(batches, schema):
    sink = pa.BufferOutputStream()
    with pa.ipc.new_stream(sink, schema) as w:
        for b in batches:
            w.write_batch(b)
    return sink.getvalue().to_pybytes()


def test_every_column_type_round_trips():
    st = AIO.SymbolTable()
    ids = np.array([st.intern(s) for s in ["b", "a", "b", "c", "a"]], dtype=np.uint32)
    cols = [np.array([1, 2, 3, 4, 4_000_000_000], np.uint32), np.array([-1, 0, 5, -7, 2], np.int32),
            np.array([1 << 40, 0, 3, 9, 2], np.uint64), np.array([-(1 << 40), 0, 3, 9, 2], np.int64),
            np.array([0.5, -0.0, np.inf, 1e-3, 2], np.float32), np.array([0.25, np.nan, -np.inf, 7, 2], np.float64), ids]
    types = [A.U32, A.I32, A.U64, A.I64, A.F32, A.F64, A.SYMBOL]
    names = ["u", "i", "U", "I", "f", "F", "s"]
    data = AIO.columns_to_ipc_stream(cols, types, names, st)
    # what any Arrow reader sees: one batch, non-nullable fields of the reference's types
    batch, = list(pa.ipc.open_stream(pa.BufferReader(data)))
    assert batch.schema.names == names and all(not f.nullable for f in batch.schema)
    assert [str(f.type) for f in batch.schema] == ["uint32", "int32", "uint64", "int64", "float", "double",
                                                    "dictionary<values=string, indices=uint32, ordered=0>"]
    assert batch.column(6).dictionary.to_pylist() == ["b", "a", "c"]          # order of first appearance
    assert batch.column(6).indices.to_pylist() == [0, 1, 0, 2, 1]
    got, gtypes, gnames = AIO.ipc_stream_to_columns(data, st)
    assert gtypes == types and gnames == names
    for g, c in zip(got, cols):
        assert g.dtype == c.dtype and g.tobytes() == c.tobytes()                # bitwise: NaN and -0.0 kept


def test_symbols_are_interned_on_import():
    arr = pa.DictionaryArray.from_arrays(pa.array([1, 0, 1], pa.uint32()), pa.array(["x", "y"]))
    batch = pa.record_batch([arr], schema=pa.schema([pa.field("s", arr.type, nullable=False)]))
    st = AIO.SymbolTable()
    st.intern("zero")
    cols, types, _ = AIO.record_batch_to_columns(batch, st)
    assert types == [A.SYMBOL]
    assert [st.resolve(int(i)) for i in cols[0]] == ["y", "x", "y"]
    assert cols[0].tolist() == [2, 1, 2] and len(st) == 3                      # ids in order of interning


def test_empty_relation_keeps_its_schema():
    data = AIO.columns_to_ipc_stream([np.zeros(0, np.uint32), np.zeros(0, np.uint64)], [A.U32, A.U64], ["a", "b"])
    cols, types, names = AIO.ipc_stream_to_columns(data)
    assert types == [A.U32, A.U64] and names == ["a", "b"] and all(len(c) == 0 for c in cols)


def test_stream_must_hold_exactly_one_batch():
    schema = pa.schema([pa.field("a", pa.uint32(), nullable=False)])
    b = pa.record_batch([pa.array([1, 2], pa.uint32())], schema=schema)
    with pytest.raises(XlbError, match="contained no record batches"):
        AIO.ipc_stream_to_columns(_stream([], schema))
    with pytest.raises(XlbError, match="multiple record batches"):
        AIO.ipc_stream_to_columns(_stream([b, b], schema))
    with pytest.raises(XlbError, match="Failed to create Arrow IPC reader"):
        AIO.ipc_stream_to_columns(b"not an arrow stream")


def test_unsupported_types_and_nulls_are_errors():
    for arr in (pa.array(["a"]), pa.array([1], pa.int8()), pa.array([1], pa.uint16())):
        batch = pa.record_batch([arr], names=["c"])
        with pytest.raises(XlbError, match="Unsupported Arrow type") as e:
            AIO.record_batch_to_columns(batch)
        assert e.value.status == A.ERR_TYPE
    batch = pa.record_batch([pa.array([1, None], pa.uint32())], names=["c"])
    with pytest.raises(XlbError, match="null values"):
        AIO.record_batch_to_columns(batch)


def test_bool_column_is_bytes_of_zero_and_one():
    data = AIO.columns_to_ipc_stream([np.array([0, 1, 7], np.uint8)], [A.BOOL])
    batch, = list(pa.ipc.open_stream(pa.BufferReader(data)))
    assert batch.column(0).to_pylist() == [False, True, True]
    cols, types, _ = AIO.ipc_stream_to_columns(data)
    assert types == [A.BOOL] and cols[0].tolist() == [0, 1, 1]


def test_symbol_table():
    st = AIO.SymbolTable()
    assert [st.intern(s) for s in ("a", "b", "a")] == [0, 1, 0] and st.resolve(1) == "b"
    with pytest.raises(KeyError):
        st.resolve(2)
    st.clear()
    assert len(st) == 0 and st.intern("b") == 0


def test_reference_export_case():
    # crates/xlog-cuda/tests/arrow_tests.rs:12-64 and :108-140: (id u32, value i64), names kept
    data = AIO.columns_to_ipc_stream([np.array([1, 2, 3, 4, 5], np.uint32), np.array([100, 200, 300, 400, 500], np.int64)],
                                     [A.U32, A.I64], ["id", "value"])
    batch, = list(pa.ipc.open_stream(pa.BufferReader(data)))
    assert (batch.num_rows, batch.num_columns) == (5, 2) and batch.schema.names == ["id", "value"]
    assert batch.schema.field(0).type == pa.uint32() and batch.schema.field(1).type == pa.int64()
    assert batch.column(0).to_pylist() == [1, 2, 3, 4, 5] and batch.column(1).to_pylist() == [100, 200, 300, 400, 500]


def test_reference_import_case():
    # crates/xlog-cuda/tests/arrow_tests.rs:210-245: a batch built by another Arrow writer
    schema = pa.schema([pa.field("x", pa.uint32(), nullable=False), pa.field("y", pa.float64(), nullable=False)])
    batch = pa.record_batch([pa.array([10, 20, 30], pa.uint32()), pa.array([1.5, 2.5, 3.5], pa.float64())], schema=schema)
    cols, types, names = AIO.ipc_stream_to_columns(_stream([batch], schema))
    assert types == [A.U32, A.F64] and names == ["x", "y"]
    assert cols[0].tolist() == [10, 20, 30] and cols[1].tolist() == [1.5, 2.5, 3.5]
