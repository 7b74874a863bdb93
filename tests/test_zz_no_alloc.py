"""The allocation-free duplicate removal, xlb_dedup_sorted_u64_static.

Some hosts cannot let a plug-in allocate device memory when they call it (their own arena owns
the GPU, or an allocation there could stall the device), so this entry point keeps its scratch in
a fixed array inside the library.  The test drives it through the C ABI with caller-owned device
buffers and checks it, bit for bit, against numpy's unique values of the same keys (independent
of this library) and against the ordinary xlb_dedup entry point, twice in a row (the second call meets the scratch the first one left behind), at a size that uses
one tile, one that needs the scan over tile counts, and one that needs the two-level scan.

The file name sorts last on purpose: if this test fails in a run that stops at the first
failure, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _sorted_keys(n, seed, distinct):
    from xlog_b200.workloads import splitmix64
    k = splitmix64(seed, 0, n) % np.uint64(distinct)
    k.sort()
    return k


@pytest.mark.parametrize("n,distinct", [(1500, 400), (300_000, 90_000), (6_000_000, 2_500_000)])
def test_static_dedup_matches_dedup_twice(provider, n, distinct):
    import torch
    from xlog_b200 import _abi as A
    from xlog_b200.lib import load

    lib = load()
    assert n <= lib.xlb_dedup_sorted_u64_static_max()
    for call in range(2):
        keys = _sorted_keys(n, 100 + call, distinct)
        # the existing entry point: full-row dedup of a one-column u64 relation
        rel = provider.create_buffer_from_slices([keys], [A.U64])
        want = provider.download(provider.dedup(rel))[0]
        # the allocation-free one, on device buffers the caller owns
        d_in = torch.from_numpy(keys.view(np.int64)).cuda()
        d_out = torch.empty(n, dtype=torch.int64, device="cuda")
        d_cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        st = lib.xlb_dedup_sorted_u64_static(C.c_void_p(d_in.data_ptr()), n, C.c_void_p(d_out.data_ptr()),
                                             C.c_void_p(d_cnt.data_ptr()), None)
        assert st == 0, lib.xlb_static_last_error().decode()
        m = int(d_cnt.item())
        got = d_out[:m].cpu().numpy().view(np.uint64)
        assert m == len(want)
        assert np.array_equal(got, np.unique(keys))   # an answer this library had no part in
        assert np.array_equal(got, want)              # and the existing entry point's; integer work: exact equality


def test_static_dedup_rejects_oversize_and_handles_empty(provider):
    import torch
    from xlog_b200 import _abi as A
    from xlog_b200.lib import load

    lib = load()
    d = torch.zeros(8, dtype=torch.int64, device="cuda")
    cnt = torch.ones(1, dtype=torch.int64, device="cuda")
    too_many = lib.xlb_dedup_sorted_u64_static_max() + 1
    st = lib.xlb_dedup_sorted_u64_static(C.c_void_p(d.data_ptr()), too_many, C.c_void_p(d.data_ptr()),
                                         C.c_void_p(cnt.data_ptr()), None)
    assert st == A.ERR_CAPACITY
    assert b"exceed" in lib.xlb_static_last_error()
    st = lib.xlb_dedup_sorted_u64_static(None, 0, None, C.c_void_p(cnt.data_ptr()), None)
    assert st == 0 and int(cnt.item()) == 0


def test_static_dedup_refuses_overlapping_buffers(provider):
    """Output blocks are written while other blocks still read their input: an output range that
    overlaps the input would race, so it is refused before anything is launched."""
    import torch
    from xlog_b200 import _abi as A
    from xlog_b200.lib import load

    lib = load()
    d = torch.arange(10_000, dtype=torch.int64, device="cuda")
    cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    for out_ptr in (d.data_ptr(), d.data_ptr() + 8 * 5000):
        st = lib.xlb_dedup_sorted_u64_static(C.c_void_p(d.data_ptr()), 6000, C.c_void_p(out_ptr), C.c_void_p(cnt.data_ptr()), None)
        assert st == A.ERR_INVALID
        assert b"overlap" in lib.xlb_static_last_error()
    assert torch.equal(d.cpu(), torch.arange(10_000, dtype=torch.int64))      # nothing was written
