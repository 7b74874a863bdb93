"""The C-ABI library without a GPU: it loads, exports every declared symbol, its structs match
the ctypes mirror, and it refuses loudly to run without a device."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import numpy as np
import pytest

from xlog_b200 import _abi as A
from xlog_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "xlb.h")


@pytest.fixture(scope="module")
def libxlb():
    if not os.path.exists(L.LIB_PATH):
        L.build()
    return L.load()


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(xlb_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound(libxlb):
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(libxlb, n), f"{n} is declared in include/xlb.h but not exported"
        assert n in L.PROTOTYPES, f"{n} has no ctypes prototype"
    for n in L.PROTOTYPES:
        assert n in names, f"{n} is bound but not declared in the header"


def test_struct_layouts_match_the_header():
    fields = {"xlb_schema": A.Schema, "xlb_config": A.Config, "xlb_node": A.Node, "xlb_rule": A.Rule,
              "xlb_scc": A.Scc, "xlb_plan": A.Plan, "xlb_run_stats": A.RunStats, "xlb_kernel_profile": A.KernelProfile}
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){"]
    for cname, ct in fields.items():
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in ct._fields_:
            lines.append(f'printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines.append("return 0;}")
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.c")
        open(src, "w").write("\n".join(lines))
        exe = os.path.join(d, "t")
        subprocess.check_call(["gcc", "-std=c99", "-o", exe, src])          # the header is plain C
        out = dict(l.split() for l in subprocess.check_output([exe], text=True).splitlines())
    for cname, ct in fields.items():
        assert int(out[cname]) == C.sizeof(ct), cname
        for fname, _ in ct._fields_:
            assert int(out[f"{cname}.{fname}"]) == getattr(ct, fname).offset, f"{cname}.{fname}"


def test_no_device_means_an_error_not_a_fallback(libxlb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from xlog_b200.provider import KernelProvider
    with pytest.raises(L.XlbError, match="no CUDA device"):
        KernelProvider()


def test_owner_function_matches_host_restatement(libxlb):
    from xlog_b200 import dist
    from xlog_b200.workloads import splitmix64
    keys = np.concatenate([splitmix64(5, 0, 2000) >> np.uint64(32), np.arange(64, dtype=np.uint64)])
    for world in (1, 2, 3, 8):
        host = dist.owner_of(keys, world)
        lib = np.array([libxlb.xlb_owner_of(int(k), world) for k in keys])
        assert np.array_equal(host, lib)


def test_plan_lowering_builds_the_c_tree():
    from xlog_b200 import programs
    cp = programs.same_generation().compile()
    assert cp.c.n_sccs == 1 and cp.c.sccs[0].n_rules == 2 and cp.c.sccs[0].is_recursive == 1
    rec = cp.c.sccs[0].rules[1]
    assert rec.head == b"sg" and rec.head_schema.arity == 2
    proj = rec.body.contents
    assert proj.kind == A.NODE_PROJECT and list(proj.cols[:2]) == [1, 5]
    j = proj.input.contents
    assert j.kind == A.NODE_JOIN and j.left_keys[0] == 3 and j.right_keys[0] == 0
    assert j.left.contents.kind == A.NODE_JOIN and j.right.contents.kind == A.NODE_SCAN
    base = cp.c.sccs[0].rules[0].body.contents.input.contents
    assert base.kind == A.NODE_FILTER and base.cmp == A.NE and base.cmp_lhs_col == 1 and base.cmp_rhs == 3


def test_rust_binding_names_every_entry_point():
    """rust/xlb-sys cannot be compiled here (no Rust toolchain); at least its extern block must
    declare every function of include/xlb.h (the two test hooks aside), with the header's flags."""
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = open(os.path.join(root, "include", "xlb.h")).read()
    rust = open(os.path.join(root, "rust", "xlb-sys", "src", "lib.rs")).read()
    declared = set(re.findall(r"^(?:xlb_status|void|const char\*|uint32_t|uint64_t)\s+(xlb_[a-z0-9_]+)\s*\(", header, re.M))
    assert len(declared) > 30
    hooks = {"xlb_comm_mark_aborted_for_test", "xlb_test_set_lookback"}
    bound = set(re.findall(r"pub fn (xlb_[a-z0-9_]+)\s*\(", rust))
    assert declared - hooks <= bound, sorted(declared - hooks - bound)
    for name, value in re.findall(r"#define (XLB_FLAG_[A-Z_]+) (\d+)u", header):
        assert re.search(rf"pub const {name}: u32 = {value};", rust), name
