"""Stop a fixpoint at the iteration limit, save (full, delta, iteration), restore into a fresh
context and resume: the result and the total number of iterations are those of an uninterrupted
run."""
import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import checkpoint as CK
from xlog_b200 import programs
from xlog_b200.executor import Executor, run_program
from xlog_b200.lib import XlbError
from xlog_b200.provider import KernelProvider

pytestmark = pytest.mark.gpu


def _executor(p, plan, edge):
    ex = Executor(p)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    if edge is not None:
        ex.put_relation("edge", p.create_buffer_from_slices(edge))
    return ex


@pytest.mark.parametrize("flags", [0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET])
@pytest.mark.parametrize("builder,out", [(programs.transitive_closure, "reach"), (programs.reach_from_source, "r")])
def test_resume_equals_an_uninterrupted_run(oracle, tmp_path, builder, out, flags):
    a = np.arange(0, 40, dtype=np.uint32)
    edge = [np.concatenate([a, [7, 20]]).astype(np.uint32), np.concatenate([a + 1, [3, 11]]).astype(np.uint32)]
    plan = builder()
    want, ex_o = oracle.run_program(plan, {"edge": edge}, [out])
    whole = KernelProvider(device=0, flags=flags)
    _, whole_stats = run_program(whole, plan, {"edge": edge}, [out])
    whole.close()

    first = KernelProvider(device=0, max_iterations=9, flags=flags | A.FLAG_KEEP_DELTAS)
    ex = _executor(first, plan, edge)
    with pytest.raises(XlbError) as e:
        ex.execute_plan(plan)
    assert e.value.status == A.ERR_ITER_LIMIT
    path = tmp_path / "tc.ckpt"
    written = CK.save(ex, ["edge", out], path, iteration=9)
    assert set(written) == {"edge", out, "__delta_" + out}
    partial = first.download(ex.get(out))
    assert 0 < len(partial[0]) < len(want[out][0])
    first.close()

    second = KernelProvider(device=0, flags=flags)
    ex2 = _executor(second, plan, None)
    assert CK.restore(ex2, path) == 9
    stats = ex2.execute_plan(plan)
    got = second.download(ex2.get(out))
    for g, w in zip(got, want[out]):
        assert np.array_equal(g, w)
    # the loop went on where it stood: no seed pass, no iteration repeated
    assert stats["iterations"] + 9 == whole_stats["iterations"]
    with pytest.raises(XlbError):
        ex2.get("__delta_" + out)          # a finished fixpoint leaves no delta behind
    second.close()


def test_without_the_flag_no_delta_is_left(oracle):
    a = np.arange(0, 30, dtype=np.uint32)
    p = KernelProvider(device=0, max_iterations=4)
    ex = _executor(p, programs.transitive_closure(), [a, a + 1])
    with pytest.raises(XlbError):
        ex.execute_plan(programs.transitive_closure())
    with pytest.raises(XlbError) as e:
        ex.get("__delta_reach")
    assert e.value.status == A.ERR_NOT_FOUND
    p.close()
