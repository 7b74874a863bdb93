"""Host-side mirror of the reference's ``Executor`` over the C ABI.

``register_relation`` / ``put_relation`` / ``execute_plan`` / ``get`` follow
crates/xlog-runtime/src/executor/mod.rs:1242, :587, :1404 and :562; the fixpoint itself runs
inside libxlb.so (``xlb_execute_plan``).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _abi as A
from .plan import ExecutionPlan
from .provider import Buffer, KernelProvider


class Executor:
    def __init__(self, provider: KernelProvider):
        self.provider = provider
        self._lib = provider._lib
        self.last_stats: dict | None = None

    def register_relation(self, rel_id: int, name: str) -> None:
        self.provider._check(self._lib.xlb_register_relation(self.provider._ctx, rel_id, name.encode()))

    def put_relation(self, name: str, buf: Buffer) -> None:
        """The store takes ownership of ``buf``."""
        self.provider._check(self._lib.xlb_store_put(self.provider._ctx, name.encode(), buf._h))
        buf.release()

    def get(self, name: str) -> Buffer:
        """Borrowed handle to a stored relation (valid until it is replaced)."""
        h = C.c_void_p()
        self.provider._check(self._lib.xlb_store_get(self.provider._ctx, name.encode(), C.byref(h)))
        return Buffer(self.provider, h, owned=False)

    def remove(self, name: str) -> None:
        self.provider._check(self._lib.xlb_store_remove(self.provider._ctx, name.encode()))

    def execute_plan(self, plan) -> dict:
        cp = plan.compile() if isinstance(plan, ExecutionPlan) else plan
        stats = A.RunStats()
        self.provider._check(self._lib.xlb_execute_plan(self.provider._ctx, C.byref(cp.c), C.byref(stats)))
        self.last_stats = stats.as_dict()
        return self.last_stats


def run_program(provider: KernelProvider, plan: ExecutionPlan, inputs: dict, outputs):
    """Register, load, execute, download: the sequence the reference's end-to-end tests use
    (crates/xlog-integration/tests/test_factorized_delta_spike.rs:202-214).
    Returns (dict name -> list of numpy columns, stats)."""
    ex = Executor(provider)
    for name, rid in plan.rel_ids.items():
        ex.register_relation(rid, name)
    for name, cols in inputs.items():
        ex.put_relation(name, provider.create_buffer_from_slices([np.asarray(c) for c in cols]))
    stats = ex.execute_plan(plan)
    return {o: provider.download(ex.get(o)) for o in outputs}, stats
