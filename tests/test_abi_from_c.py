"""The header and the library from plain C: tests/abi_example.c is compiled as strict C99 against
include/xlb.h and linked with libxlb.so.  Without a GPU the program must fail loudly at
xlb_ctx_create (no fallback); with one it must print the reference's known answer."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def example(tmp_path_factory):
    if not shutil.which("gcc"):
        pytest.skip("no C compiler")
    import __graft_entry__ as g
    g.build()
    exe = str(tmp_path_factory.mktemp("abi") / "abi_example")
    cmd = ["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I" + os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "abi_example.c"), "-L" + os.path.join(ROOT, "xlog_b200"), "-lxlb",
           "-Wl,-rpath," + os.path.join(ROOT, "xlog_b200"), "-o", exe]
    p = subprocess.run(cmd, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr
    return exe


def test_header_is_c99_and_no_device_is_an_error(example):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the GPU test runs the program")
    p = subprocess.run([example], capture_output=True, text=True, timeout=120)
    assert p.returncode == 10 and "xlb_ctx_create" in p.stderr      # XLB_ERR_CUDA, reported, nothing computed
    assert "ok" not in p.stdout


@pytest.mark.gpu
def test_c_program_gets_the_known_answer(example):
    p = subprocess.run([example], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "reach: 6 rows" in p.stdout and p.stdout.strip().endswith("ok")
