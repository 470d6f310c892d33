"""Numerics of single device kernels against plain PyTorch references."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rows(n, groups, nbins, seed=0, stride=None):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    stride = stride or ((groups + 4 + 15) // 16) * 16
    rows = torch.zeros((n, stride), dtype=torch.uint8, device="cuda")
    for k, nb in enumerate(nbins):
        rows[:, k] = torch.randint(0, nb, (n,), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    return rows


def _ref_hist(rows, nbins, g, h, idx=None):
    sel = rows if idx is None else rows[idx.long()]
    gg = g if idx is None else g[idx.long()]; hh = h if idx is None else h[idx.long()]
    total = int(sum(nbins)); out = torch.zeros((total, 2), dtype=torch.float64, device="cuda")
    off = 0
    for k, nb in enumerate(nbins):
        b = sel[:, k].long() + off
        out[:, 0].index_add_(0, b, gg.double()); out[:, 1].index_add_(0, b, hh.double())
        off += nb
    return out


@pytest.mark.parametrize("n,groups,nb,qbins,rpb", [(1, 1, 2, 4, 512), (33, 3, 16, 4, 512), (1023, 28, 64, 4, 512), (50000, 28, 64, 4, 8192), (30000, 40, 16, 64, 8192), (40000, 7, 255, 64, 4096), (20000, 130, 255, 16, 2048)])
@pytest.mark.parametrize("lane_mode", [0, 1, 2])
def test_hist_quant_exact(n, groups, nb, qbins, rpb, lane_mode):
    from falcata_b200 import ops
    nbins = [nb] * groups
    rows = _rows(n, groups, nbins)
    g = torch.Generator(device="cuda"); g.manual_seed(1)
    gi = torch.randint(-qbins // 2, qbins // 2 + 1, (n,), generator=g, device="cuda", dtype=torch.int32)
    hi = torch.randint(0, qbins + 1, (n,), generator=g, device="cuda", dtype=torch.int32)
    packed = (gi << 16) | (hi & 0xFFFF)
    ref = _ref_hist(rows, nbins, gi, hi)
    out = ops.histogram(rows, packed, nbins, quant=True, quant_bins=qbins, rows_per_block=rpb, lane_mode=lane_mode)
    assert torch.equal(out, ref.long())
    idx = torch.randperm(n, generator=g, device="cuda")[: max(1, n // 3)].int().sort().values
    out = ops.histogram(rows, packed, nbins, idx=idx, quant=True, quant_bins=qbins, rows_per_block=rpb, lane_mode=lane_mode)
    assert torch.equal(out, _ref_hist(rows, nbins, gi, hi, idx).long())


@pytest.mark.parametrize("n,nb,qbins", [(1, 64, 4), (33, 64, 4), (1023, 64, 4), (50000, 64, 4), (300001, 64, 64), (70000, 16, 4), (40000, 37, 100)])
@pytest.mark.parametrize("groups", [28, 32, 5])
def test_hist_tensor_core_exact(n, nb, qbins, groups):
    """The one-hot tcgen05 instance (lane_mode 3: int8 MMA, int32 accumulators in tensor memory, TMA-fed row tiles)
    gives the exact integer histogram, like the SIMT instances: root-level shape, 32-byte rows."""
    from falcata_b200 import ops
    nbins = [nb] * groups
    rows = _rows(n, groups, nbins, stride=32)
    rows[:, groups:] = 201          # bytes past the last group are not bins: the kernel must ignore them
    g = torch.Generator(device="cuda"); g.manual_seed(2)
    gi = torch.randint(-(qbins // 2), qbins // 2 + 1, (n,), generator=g, device="cuda", dtype=torch.int32)
    hi = torch.randint(0, qbins + 1, (n,), generator=g, device="cuda", dtype=torch.int32)
    packed = (gi << 16) | (hi & 0xFFFF)
    ref = _ref_hist(rows, nbins, gi, hi)
    out = ops.histogram(rows, packed, nbins, quant=True, quant_bins=qbins, lane_mode=3)
    assert torch.equal(out, ref.long())
    # same answer as the lane kernel on the same input
    assert torch.equal(out, ops.histogram(rows, packed, nbins, quant=True, quant_bins=qbins, rows_per_block=8192, lane_mode=1))


def test_hist_quant_gh_in_row():
    from falcata_b200 import ops
    n, groups = 5000, 28
    nbins = [64] * groups
    rows = _rows(n, groups, nbins)
    gi = torch.randint(-2, 3, (n,), device="cuda", dtype=torch.int32); hi = torch.randint(0, 5, (n,), device="cuda", dtype=torch.int32)
    packed = (gi << 16) | (hi & 0xFFFF)
    rows.view(torch.int32).view(n, -1)[:, -1] = packed      # last 4 bytes of every 32-byte row
    gh_view = rows.view(-1)[rows.shape[1] - 4:]
    out = ops.histogram(rows, gh_view, nbins, quant=True, quant_bins=4, gh_stride=rows.shape[1], count=n)
    assert torch.equal(out, _ref_hist(rows, nbins, gi, hi).long())


@pytest.mark.parametrize("n,groups,nb", [(1, 1, 2), (33, 3, 16), (30000, 20, 100), (50000, 28, 64), (70001, 100, 255), (20000, 130, 256)])
@pytest.mark.parametrize("lane_mode", [0, 1, 2])
def test_hist_float_close(n, groups, nb, lane_mode):
    """fp32 gradients: the flat shared-atomic instance (0) and the lane instance in its load-add-store (1) and
    reduction-add (2) forms, whole data set and a row subset, against float64 sums."""
    from falcata_b200 import ops
    nbins = [nb] * groups
    rows = _rows(n, groups, nbins)
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    gh = torch.randn(n, 2, device="cuda", generator=g); gh[:, 1].abs_()
    ref = _ref_hist(rows, nbins, gh[:, 0], gh[:, 1])
    out = ops.histogram(rows, gh.contiguous(), nbins, quant=False, lane_mode=lane_mode, rows_per_block=8192)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-3)
    idx = torch.randperm(n, generator=g, device="cuda")[: max(1, n // 3)].int().sort().values
    out = ops.histogram(rows, gh.contiguous(), nbins, idx=idx, quant=False, lane_mode=lane_mode, rows_per_block=8192)
    torch.testing.assert_close(out, _ref_hist(rows, nbins, gh[:, 0], gh[:, 1], idx), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("stochastic", [True, False])
def test_quantize_matches_reference(stochastic):
    from falcata_b200 import ops
    n, bins = 200000, 4
    torch.manual_seed(0)
    g = torch.randn(n, device="cuda"); h = torch.rand(n, device="cuda")
    packed, scales, sums = ops.quantize(g, h, bins, stochastic, seed=7, iter_key=3)
    gs = g.abs().max() / (bins // 2); hs = h.abs().max() / bins
    torch.testing.assert_close(scales, torch.stack([gs, hs]))
    gi = packed >> 16; hi = packed & 0xFFFF
    assert int(gi.abs().max()) <= bins // 2 + 1 and int(hi.max()) <= bins + 1 and int(hi.min()) >= 0
    assert torch.equal(sums, torch.stack([gi.long().sum(), hi.long().sum()]))
    if not stochastic:
        ref_g = torch.trunc(torch.addcmul(torch.where(g >= 0, 0.5, -0.5), g, (1.0 / gs).expand_as(g))).int()
        assert (ref_g != gi).float().mean() < 1e-3     # fused vs unfused rounding may differ on exact ties only
    else:
        # unbiased: E[q * scale] = g (the mean error over 200k rows has a standard deviation of about 0.002)
        assert abs(float((gi.float() * gs - g).mean())) < 0.02
    p2, _, _ = ops.quantize(g, h, bins, stochastic, seed=7, iter_key=3)
    assert torch.equal(packed, p2)


@pytest.mark.parametrize("n", [1, 31, 2048, 2049, 100000])
def test_partition_stable(n):
    from falcata_b200 import ops
    rows = _rows(max(n, 8) * 2, 4, [64] * 4)
    idx = torch.randperm(rows.shape[0], device="cuda")[:n].int().sort().values
    out, left = ops.partition(rows, idx, group=2, threshold=20)
    b = rows[idx.long(), 2]
    ref = torch.cat([idx[b <= 20], idx[b > 20]])
    assert left == int((b <= 20).sum()) and torch.equal(out, ref)
    out, left = ops.partition(rows, idx, group=1, threshold=10, default_left=False, missing_type=1, default_bin=3)
    b = rows[idx.long(), 1]
    goes_left = (b <= 10) & (b != 3)
    assert torch.equal(out, torch.cat([idx[goes_left], idx[~goes_left]]))


def test_cross_rank_wait_is_bounded_and_reports_status():
    # failure detection on the device: a wait on a flag that nothing sets must run out of its spin budget,
    # record the timeout status for the host and return (the context stays usable afterwards)
    from falcata_b200 import ops

    status, seen = ops.bounded_wait_probe(2000)
    assert status == 1 and seen == 0
    x = torch.ones(8, device="cuda")
    assert float(x.sum().item()) == 8.0


def test_symmetric_heap_guard_words_catch_an_overrun():
    """FALCATA_DEBUG=canary puts a guard block behind every region carved from the symmetric heap; a write past a region
    (made here from the host with a memset inside the heap, so nothing faults) is reported with the region's index."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    code = (
        "import ctypes, torch, falcata_b200 as fb\n"
        "from falcata_b200.basic import _lib\n"
        "lib = _lib()\n"
        "torch.cuda.init(); torch.zeros(1, device='cuda')\n"
        "h = ctypes.create_string_buffer(64)\n"
        "assert lib.FB_FabricCreate(0, 1, ctypes.c_int64(1 << 20), h) == 0\n"
        "assert lib.FB_FabricConnect(h) == 0\n"
        "a = ctypes.c_int64(); b = ctypes.c_int64(); bad = ctypes.c_int(7)\n"
        "assert lib.FB_FabricDebugAlloc(ctypes.c_int64(1000), ctypes.byref(a)) == 0\n"
        "assert lib.FB_FabricDebugAlloc(ctypes.c_int64(4096), ctypes.byref(b)) == 0\n"
        "assert b.value >= a.value + 1000 + 256\n"
        "assert lib.FB_FabricDebugFill(ctypes.c_int64(a.value), ctypes.c_int64(1000), 1) == 0\n"
        "assert lib.FB_FabricCheckCanaries(ctypes.byref(bad)) == 0 and bad.value == -1\n"
        "assert lib.FB_FabricDebugFill(ctypes.c_int64(b.value), ctypes.c_int64(4100), 2) == 0\n"
        "assert lib.FB_FabricCheckCanaries(ctypes.byref(bad)) == 0\n"
        "print('BROKEN', bad.value)\n"
        "lib.FB_FabricDestroy()\n")
    env = dict(os.environ, FALCATA_DEBUG="canary", PYTHONPATH=str(Path(__file__).resolve().parents[1]))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
    assert "BROKEN 2" in out.stdout   # region 0 is the heap's own all-reduce area, 1 and 2 the two carved here
