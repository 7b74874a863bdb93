"""Arrow IPC streams on either side of the fixpoint: relations read from stream files, a program
run on them, the result written back and read by a plain Arrow reader."""
import numpy as np
import pyarrow as pa
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import arrow_io as AIO
from xlog_b200 import programs, workloads
from xlog_b200.executor import Executor
from xlog_b200.lib import XlbError

pytestmark = pytest.mark.gpu


def test_relation_round_trips_through_a_stream_file(provider, tmp_path):
    cols = [np.array([5, 1, 5, 9], np.uint32), np.array([-3, 7, -3, 0], np.int64), np.array([0.5, 2.0, 0.5, -1.0], np.float64)]
    buf = provider.create_buffer_from_slices(cols, [A.U32, A.I64, A.F64])
    path = tmp_path / "rel.arrow"
    AIO.write_arrow_ipc_stream_file(provider, buf, path, ["k", "v", "w"])
    back = AIO.read_arrow_ipc_stream_file(provider, path)
    assert back.schema() == [A.U32, A.I64, A.F64]
    for g, c in zip(provider.download(back), cols):
        assert np.array_equal(g, c)
    # the operators take what was read: dedup of the imported relation
    uniq = provider.download(provider.dedup(back))
    assert [c.tolist() for c in uniq] == [[1, 5, 9], [7, -3, 0], [2.0, 0.5, -1.0]]


def test_empty_stream_gives_an_empty_relation_of_the_schema(provider):
    data = AIO.columns_to_ipc_stream([np.zeros(0, np.uint32), np.zeros(0, np.uint32)], [A.U32, A.U32])
    buf = AIO.from_arrow_ipc_stream(provider, data)
    assert buf.num_rows() == 0 and buf.schema() == [A.U32, A.U32]


def test_fixpoint_from_arrow_inputs_to_arrow_output(provider, oracle, tmp_path):
    c0, c1 = workloads.uniform_digraph(200, 600, 4)
    (tmp_path / "edge.arrow").write_bytes(AIO.columns_to_ipc_stream([c0, c1], [A.U32, A.U32], ["src", "dst"]))
    plan = programs.transitive_closure()
    ex = Executor(provider)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    ex.put_relation("edge", AIO.read_arrow_ipc_stream_file(provider, tmp_path / "edge.arrow"))
    ex.execute_plan(plan)
    AIO.write_arrow_ipc_stream_file(provider, ex.get("reach"), tmp_path / "reach.arrow", ["x", "y"])
    batch, = list(pa.ipc.open_stream(pa.OSFile(str(tmp_path / "reach.arrow"))))
    want, _ = oracle.run_program(plan, {"edge": [c0, c1]}, ["reach"])
    assert np.array_equal(batch.column(0).to_numpy(), want["reach"][0])
    assert np.array_equal(batch.column(1).to_numpy(), want["reach"][1])


def test_missing_file_is_reported(provider, tmp_path):
    with pytest.raises(XlbError, match="Failed to read Arrow IPC stream from"):
        AIO.read_arrow_ipc_stream_file(provider, tmp_path / "nothing.arrow")


def test_imported_plan_runs_on_the_gpu(oracle):
    # the caller side: a serialized plan (as the reference's planner would print it) drives the executor
    from test_plan_json_cpu import TC_JSON
    from xlog_b200 import plan_json as PJ
    from xlog_b200.executor import run_program
    from xlog_b200.provider import KernelProvider
    plan = PJ.plan_from_json(TC_JSON, rel_names={0: "edge", 1: "reach"})
    c0, c1 = workloads.uniform_digraph(150, 400, 9)
    fresh = KernelProvider(device=0)      # its own store: `reach` must start empty
    got, stats = run_program(fresh, plan, {"edge": [c0, c1]}, ["reach"])
    fresh.close()
    want, ex = oracle.run_program(programs.transitive_closure(), {"edge": [c0, c1]}, ["reach"])
    assert all(np.array_equal(g, w) for g, w in zip(got["reach"], want["reach"]))
    assert stats["candidate_tuples"] == ex.candidates
