"""xlog_b200 — B200-native semi-naive Datalog fixpoint data plane.

The product is ``libxlb.so`` (hand-written sm_100a CUDA behind the C ABI of include/xlb.h).
This package is the thin host-side mirror of the reference's provider / executor interface
used by the tests and the benchmark, plus the seeded workload generators.
"""
from . import _abi as abi  # noqa: F401
from .lib import XlbError, build, load  # noqa: F401
from .plan import CompiledRule, ExecutionPlan, Filter, Join, Project, Scan, Scc, Union  # noqa: F401


def __getattr__(name):
    if name in ("KernelProvider", "Buffer"):
        from . import provider
        return getattr(provider, name)
    if name in ("Executor", "run_program"):
        from . import executor
        return getattr(executor, name)
    raise AttributeError(name)
