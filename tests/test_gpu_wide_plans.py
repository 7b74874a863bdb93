"""Plans over u64, signed and floating columns: the executor runs them on dictionary ranks and
decodes the heads; results must equal the CPU oracle's, in the typed order, and the store must hold
the caller's relations again afterwards."""
import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import programs
from xlog_b200.executor import Executor, run_program
from xlog_b200.lib import XlbError
from xlog_b200.plan import CompiledRule, ExecutionPlan, Filter, Scan, Scc
from xlog_b200.provider import KernelProvider

pytestmark = pytest.mark.gpu
HI = 1 << 32


def _typed(plan, t):
    for s in plan.sccs:
        for r in s.rules:
            r.head_types = tuple(t for _ in r.head_types)
    return plan


def _same(got, want):
    assert len(got) == len(want)
    for g, w in zip(got, want):
        assert g.dtype == w.dtype and g.tobytes() == w.tobytes()


def test_u64_three_cycle_gives_all_nine_pairs(oracle):
    # crates/xlog-integration/tests/test_factorized_delta_e2e.rs:385-411
    edge = [np.array([HI, HI + 1, HI + 2], np.uint64), np.array([HI + 1, HI + 2, HI], np.uint64)]
    plan = _typed(programs.transitive_closure(), A.U64)
    p = KernelProvider(device=0)
    ex = Executor(p)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    ex.put_relation("edge", p.create_buffer_from_slices(edge, [A.U64, A.U64]))
    ex.execute_plan(plan)
    reach = ex.get("reach")
    assert reach.schema() == [A.U64, A.U64] and reach.is_canonical()
    got = p.download(reach)
    assert list(zip(*[c.tolist() for c in got])) == [(HI + a, HI + b) for a in range(3) for b in range(3)]
    # the caller's relation is back in the store, untouched
    back = ex.get("edge")
    assert back.schema() == [A.U64, A.U64]
    _same(p.download(back), edge)
    p.close()


@pytest.mark.parametrize("flags", [0, A.FLAG_NO_DENSE, A.FLAG_NO_DENSE | A.FLAG_NO_TUPLE_SET])
@pytest.mark.parametrize("dtype,code", [(np.uint64, A.U64), (np.int64, A.I64), (np.int32, A.I32), (np.float64, A.F64)])
def test_typed_closure_against_the_oracle(oracle, dtype, code, flags):
    rng = np.random.default_rng(11)
    ids = rng.integers(0, 60, size=(2, 150))
    if np.dtype(dtype).kind == "u":
        vals = (ids.astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15)) | np.uint64(1 << 40)
    elif np.dtype(dtype).kind == "i":
        vals = (ids - 30) * (1000 if dtype == np.int32 else 10 ** 12)
    else:
        vals = (ids - 30) * 0.25
    edge = [vals[0].astype(dtype), vals[1].astype(dtype)]
    plan = _typed(programs.transitive_closure(), code)
    p = KernelProvider(device=0, flags=flags)
    got, stats = run_program_typed(p, plan, {"edge": (edge, [code, code])}, ["reach"])
    want, ex = oracle.run_program(plan, {"edge": edge}, ["reach"])
    _same(got["reach"], want["reach"])
    assert stats["candidate_tuples"] == ex.candidates
    p.close()


def run_program_typed(p, plan, inputs, outputs):
    ex = Executor(p)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    for name, (cols, types) in inputs.items():
        ex.put_relation(name, p.create_buffer_from_slices(cols, types))
    stats = ex.execute_plan(plan)
    return {o: p.download(ex.get(o)) for o in outputs}, stats


def test_constants_become_rank_bounds(oracle):
    rng = np.random.default_rng(5)
    e = [(rng.integers(0, 40, 300).astype(np.uint64) << np.uint64(33)) + np.uint64(7), rng.integers(0, 40, 300).astype(np.uint64) << np.uint64(33)]
    ids = {"e": 0, "h": 1}
    present, absent = int(e[1][3]), (5 << 33) + 1
    for op in (A.EQ, A.NE, A.LT, A.LE, A.GT, A.GE):
        for const in (present, absent, 0, (1 << 64) - 1):
            plan = ExecutionPlan([Scc(0, False, [CompiledRule("h", Filter(Scan(0), op, 1, const, True), (A.U64, A.U64))])], ids)
            p = KernelProvider(device=0)
            got, _ = run_program_typed(p, plan, {"e": (e, [A.U64, A.U64])}, ["h"])
            want, _ = oracle.run_program(plan, {"e": e}, ["h"])
            _same(got["h"], want["h"])
            p.close()


def test_reach_from_a_u64_source(oracle):
    a = np.arange(0, 30, dtype=np.uint64) + np.uint64(HI)
    edge = [a, a + np.uint64(1)]
    plan = programs.reach_from_source(int(HI))
    for s in plan.sccs:
        for r in s.rules:
            r.head_types = (A.U64,)
    p = KernelProvider(device=0)
    got, _ = run_program_typed(p, plan, {"edge": (edge, [A.U64, A.U64])}, ["r"])
    want, _ = oracle.run_program(plan, {"edge": edge}, ["r"])
    _same(got["r"], want["r"])
    assert len(got["r"][0]) == 30
    p.close()


def test_failure_puts_the_callers_relations_back():
    a = np.arange(0, 40, dtype=np.uint64) + np.uint64(HI)
    plan = _typed(programs.transitive_closure(), A.U64)
    p = KernelProvider(device=0, max_iterations=2)
    ex = Executor(p)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    ex.put_relation("edge", p.create_buffer_from_slices([a, a + np.uint64(1)], [A.U64, A.U64]))
    with pytest.raises(XlbError) as e:
        ex.execute_plan(plan)
    assert e.value.status == A.ERR_ITER_LIMIT
    assert ex.get("edge").schema() == [A.U64, A.U64]
    _same(p.download(ex.get("edge")), [a, a + np.uint64(1)])
    with pytest.raises(XlbError) as e:
        ex.get("reach")                      # no half-finished relation of ranks is left behind
    assert e.value.status == A.ERR_NOT_FOUND
    p.close()
