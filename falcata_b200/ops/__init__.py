"""Kernel-level entry points (one function per device kernel) used by the numerics tests.

Every function takes torch CUDA tensors, runs exactly one kernel of the training path through the
native library and returns torch tensors. If the native library is missing these raise: there is
no PyTorch fallback on this path.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from ..basic import _lib


def _check(ret: int) -> None:
    if ret != 0:
        lib = _lib()
        lib.FB_OpsLastError.restype = ctypes.c_char_p
        raise RuntimeError(lib.FB_OpsLastError().decode())


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def histogram(rows: torch.Tensor, gh: torch.Tensor, group_num_bin: Sequence[int], idx: Optional[torch.Tensor] = None, quant: bool = True, quant_bins: int = 4,
              rows_per_block: int = 2048, max_part_bins: int = 6144, gh_stride: Optional[int] = None, count: Optional[int] = None, lane_mode: int = 0) -> torch.Tensor:
    """Per-bin (grad, hess) sums of the selected rows. ``rows``: uint8 [n, stride]; ``gh``: int32 packed (quant) or float32 [n, 2]."""
    assert rows.is_cuda and rows.dtype == torch.uint8 and rows.is_contiguous()
    g = np.ascontiguousarray(np.asarray(group_num_bin, dtype=np.int32))
    total = int(g.sum())
    n = int(count if count is not None else (idx.numel() if idx is not None else rows.shape[0]))
    out = torch.zeros((total, 2), dtype=torch.int64 if quant else torch.float64, device=rows.device)
    stride = gh_stride if gh_stride is not None else (4 if quant else 8)
    _check(_lib().FB_OpHistogram(_p(rows), rows.shape[1], len(g), _p(gh), stride, _p(idx), n, g.ctypes.data_as(ctypes.c_void_p), 1 if quant else 0, quant_bins,
                                  rows_per_block, max_part_bins, lane_mode, _p(out)))
    return out


def quantize(grad: torch.Tensor, hess: torch.Tensor, bins: int, stochastic: bool, seed: int, iter_key: int, row_offset: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    n = grad.numel()
    packed = torch.empty(n, dtype=torch.int32, device=grad.device)
    scales = torch.empty(2, dtype=torch.float32, device=grad.device)
    sums = torch.empty(2, dtype=torch.int64, device=grad.device)
    _check(_lib().FB_OpQuantize(_p(grad), _p(hess), n, bins, 1 if stochastic else 0, ctypes.c_uint(seed), ctypes.c_uint(iter_key), ctypes.c_ulonglong(row_offset),
                                 _p(packed), _p(scales), _p(sums)))
    return packed, scales, sums


def partition(rows: torch.Tensor, idx: torch.Tensor, group: int, threshold: int, default_left: bool = True, missing_type: int = 0, default_bin: int = 0,
              num_bin: int = 256) -> Tuple[torch.Tensor, int]:
    out = torch.empty_like(idx)
    left = ctypes.c_int(0)
    _check(_lib().FB_OpPartition(_p(rows), rows.shape[1], _p(idx), idx.numel(), group, threshold, 1 if default_left else 0, missing_type, default_bin, num_bin, _p(out), ctypes.byref(left)))
    return out, left.value


def launch_count() -> int:
    out = ctypes.c_longlong(0)
    _lib().FB_OpLaunchCount(ctypes.byref(out))
    return out.value


def bounded_wait_probe(max_spins: int = 1000):
    """Run the kernels' cross-rank wait on a flag that nothing sets. Returns (status word, flag seen): the
    wait must give up after ``max_spins`` polls and report status 1 (wait timeout) without hanging."""
    st, seen = ctypes.c_int(-1), ctypes.c_int(-1)
    if _lib().FB_OpBoundedWaitProbe(ctypes.c_longlong(int(max_spins)), ctypes.byref(st), ctypes.byref(seen)) != 0:
        _lib().FB_OpsLastError.restype = ctypes.c_char_p
        raise RuntimeError(_lib().FB_OpsLastError().decode())
    return st.value, seen.value
