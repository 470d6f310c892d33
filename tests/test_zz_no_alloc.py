"""The allocation-free partition entry point against the ordinary one.

Some callers of this library cannot allocate device memory while they work (a host callback running
inside a captured stream, a latency-bound serving thread that must stay clear of the CUDA allocator,
a process pinned to a fixed memory budget). For them the library exports one C function whose
scratch space is a fixed array inside the library image. This test calls that function through its
exported C symbol, twice in a row with different inputs (the shared scratch keeps the first call's
leftovers), and checks both results against FB_OpPartition, which allocates its scratch buffers.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rows(n, groups=6, nb=64, seed=0):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    rows = torch.zeros((n, 16), dtype=torch.uint8, device="cuda")
    rows[:, :groups] = torch.randint(0, nb, (n, groups), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    return rows


def _no_alloc_partition(lib, rows, idx, group, threshold, default_left, missing_type, default_bin, num_bin):
    out = torch.empty_like(idx)
    left = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.FB_OpPartitionNoAlloc(ctypes.c_void_p(rows.data_ptr()), rows.shape[1], ctypes.c_void_p(idx.data_ptr()), idx.numel(), group, threshold,
                                   1 if default_left else 0, missing_type, default_bin, num_bin, ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(left.data_ptr()),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        lib.FB_NoAllocLastError.restype = ctypes.c_char_p
        raise RuntimeError(lib.FB_NoAllocLastError().decode())
    torch.cuda.synchronize()
    return out, int(left.item())


def test_no_alloc_partition_matches_allocating_entry_twice():
    from falcata_b200 import ops
    from falcata_b200.basic import _lib

    lib = _lib()
    cases = [  # (rows, picked rows, group, threshold, default_left, missing_type, default_bin)
        (_rows(300000, seed=1), 0.5, 2, 20, True, 0, 0),
        (_rows(70001, seed=2), 0.9, 4, 41, False, 1, 7),     # second call: fewer rows, other column, zero-as-missing routing
    ]
    for rows, frac, group, thr, dl, mt, db in cases:
        n = rows.shape[0]
        idx = torch.randperm(n, device="cuda")[: int(n * frac)].int().sort().values.contiguous()
        ref_out, ref_left = ops.partition(rows, idx, group=group, threshold=thr, default_left=dl, missing_type=mt, default_bin=db, num_bin=64)
        got_out, got_left = _no_alloc_partition(lib, rows, idx, group, thr, dl, mt, db, 64)
        assert got_left == ref_left
        assert torch.equal(got_out, ref_out)      # integer row ids: exact equality, as in the other partition tests


def test_no_alloc_partition_at_the_largest_size_and_with_no_rows():
    """The two ends of the accepted range: every chunk counter of the fixed scratch array in use, and none."""
    from falcata_b200 import ops
    from falcata_b200.basic import _lib

    lib = _lib()
    n = 1 << 22
    rows = _rows(n, seed=3)
    idx = torch.arange(n, dtype=torch.int32, device="cuda")
    ref_out, ref_left = ops.partition(rows, idx, group=1, threshold=30, default_left=True, missing_type=0, default_bin=0, num_bin=64)
    got_out, got_left = _no_alloc_partition(lib, rows, idx, 1, 30, True, 0, 0, 64)
    assert got_left == ref_left and torch.equal(got_out, ref_out)
    empty = idx[:0].contiguous()
    got_out, got_left = _no_alloc_partition(lib, rows, empty, 1, 30, True, 0, 0, 64)
    assert got_left == 0 and got_out.numel() == 0


def test_no_alloc_partition_rejects_bad_arguments():
    from falcata_b200.basic import _lib

    lib = _lib()
    lib.FB_NoAllocLastError.restype = ctypes.c_char_p
    rows = _rows(16)
    idx = torch.zeros(16, dtype=torch.int32, device="cuda")
    out = torch.empty_like(idx); left = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = lambda group, idx_ptr: (ctypes.c_void_p(rows.data_ptr()), 16, ctypes.c_void_p(idx_ptr), 16, group, 1, 1, 0, 0, 64,
                                   ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(left.data_ptr()), ctypes.c_void_p(0))
    assert lib.FB_OpPartitionNoAlloc(*args(16, idx.data_ptr())) == -1 and b"feature group" in lib.FB_NoAllocLastError()
    assert lib.FB_OpPartitionNoAlloc(*args(-1, idx.data_ptr())) == -1
    assert lib.FB_OpPartitionNoAlloc(*args(0, 0)) == -1 and b"null buffer" in lib.FB_NoAllocLastError()


def test_no_alloc_partition_rejects_oversized_call():
    from falcata_b200.basic import _lib

    lib = _lib()
    rows = _rows(16)
    idx = torch.zeros(16, dtype=torch.int32, device="cuda")
    out = torch.empty_like(idx); left = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.FB_OpPartitionNoAlloc(ctypes.c_void_p(rows.data_ptr()), 16, ctypes.c_void_p(idx.data_ptr()), (1 << 22) + 1, 0, 1, 1, 0, 0, 64,
                                   ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(left.data_ptr()), ctypes.c_void_p(0))
    assert rc == -1
    lib.FB_NoAllocLastError.restype = ctypes.c_char_p
    assert b"at most" in lib.FB_NoAllocLastError()
