"""Failure reporting without a GPU fault: a bounded device-side wait that runs out, and the state
of a context whose communicator was aborted.

The one-sweep radix sort lets a tile wait for the tiles before it.  Every such wait has a poll
limit; a tile that reaches it publishes XLB_ERR_TIMEOUT in the device status word and returns.
The test makes the wait run out on purpose, by a flag that nothing sets: with the test knob the
tiles take their numbers from 1, so tile 0 never runs and never publishes its counts.  The kernel
ends by itself within microseconds (the limit is set to a few thousand polls), the operator call
fails with XLB_ERR_TIMEOUT instead of returning a wrong relation, and the next call on the same
context is clean.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_lookback_wait_runs_out_and_the_context_stays_usable():
    from xlog_b200 import _abi as A
    from xlog_b200.lib import XlbError
    from xlog_b200.provider import KernelProvider
    from xlog_b200.workloads import splitmix64

    prov = KernelProvider(device=0)
    try:
        keys = splitmix64(5, 0, 200_000) % np.uint64(1 << 40)       # 49 tiles of 4096 keys, five varying digits
        rel = prov.create_buffer_from_slices([keys], [A.U64])
        prov._check(prov._lib.xlb_test_set_lookback(prov._ctx, 4000, 1))
        with pytest.raises(XlbError) as e:
            prov.sort(rel, [0])
        assert e.value.status == A.ERR_TIMEOUT
        with pytest.raises(XlbError) as e:                            # dedup sorts first: the same report, not a short relation
            prov.dedup(rel)
        assert e.value.status == A.ERR_TIMEOUT
        prov._check(prov._lib.xlb_test_set_lookback(prov._ctx, 0, 0))
        got = prov.download(prov.sort(rel, [0]))[0]
        assert np.array_equal(got, np.sort(keys))                     # the status word was cleared with the report
        got = prov.download(prov.dedup(rel))[0]
        assert np.array_equal(got, np.unique(keys))
    finally:
        prov.close()


def test_calls_after_a_communicator_abort_fail_at_once():
    """After an exchange timed out the communicator is gone; a later plan over several ranks must
    say so instead of handing a null communicator to NCCL.  No peer and no collective is involved:
    the hook only records the state an abort leaves behind."""
    from xlog_b200 import _abi as A, programs, workloads
    from xlog_b200.executor import Executor
    from xlog_b200.lib import XlbError
    from xlog_b200.provider import KernelProvider

    prov = KernelProvider(device=0)
    try:
        prov._check(prov._lib.xlb_comm_mark_aborted_for_test(prov._ctx))
        c0, c1 = workloads.uniform_digraph(50, 120, 3)
        plan = programs.transitive_closure()
        ex = Executor(prov)
        for name, rid in plan.rel_ids.items():
            ex.register_relation(rid, name)
        ex.put_relation("edge", prov.create_buffer_from_slices([c0, c1]))
        with pytest.raises(XlbError) as e:
            ex.execute_plan(plan)
        assert e.value.status == A.ERR_NCCL
        assert "aborted" in e.value.message
        # operators that need no other rank still work on this context
        got = prov.download(prov.dedup(prov.create_buffer_from_slices([c0, c1])))
        order = np.lexsort((c1, c0))
        assert np.array_equal(got[0], c0[order]) and np.array_equal(got[1], c1[order])
    finally:
        prov.close()
