"""Rank bootstrap and host-side collectives.

``torch.distributed`` is used only for plumbing: exchanging the bin-construction sample, CUDA IPC
handles of the symmetric heap, and (for the CPU learners) the injected all-reduce / all-gather.
Parity: include/Falcata/cuda/cuda_nccl_topology.hpp:L121-185 (communicator bootstrap),
src/c_api.cpp:L3218 (FLC_NetworkInitWithFunctions), src/io/dataset_loader.cpp:L672-759
(distributed bin finding).
"""
from __future__ import annotations

import ctypes
from typing import Any, Tuple

import numpy as np

_CALLBACKS: list = []


def _dist():
    import torch.distributed as dist

    return dist if dist.is_available() and dist.is_initialized() else None


def world() -> Tuple[int, int]:
    d = _dist()
    return (d.get_rank(), d.get_world_size()) if d else (0, 1)


def gather_bin_sample(t: Any, sample_cnt: int, seed: int) -> Tuple[np.ndarray, int]:
    """Rows used to find bin boundaries: a seeded sample of this rank's rows, concatenated over ranks
    so that every rank derives identical bin mappers. Returns (sample [ns, ncol] float64, total rows)."""
    import torch

    rank, ws = world()
    n = t.shape[0]
    total = n
    d = _dist()
    if d and ws > 1:
        cnt = torch.tensor([n], dtype=torch.int64, device=t.device if t.is_cuda and d.get_backend() == "nccl" else "cpu")
        d.all_reduce(cnt)
        total = int(cnt.item())
    take = min(n, max(1, int(round(sample_cnt * (n / max(1, total))))))
    g = torch.Generator(device="cpu"); g.manual_seed(seed * 7919 + rank)
    idx = torch.randperm(n, generator=g)[:take].sort().values if take < n else torch.arange(n)
    local = t[idx.to(t.device)].to(torch.float64).cpu().numpy()
    if d and ws > 1:
        parts = [None] * ws
        d.all_gather_object(parts, local)
        local = np.concatenate(parts, axis=0)
    return local, total


def init_host_network() -> None:
    """Inject torch.distributed (gloo or nccl-with-cpu-staging) collectives into the native host learners."""
    import torch

    from ..basic import _lib, _safe_call

    d = _dist()
    if d is None or d.get_world_size() == 1:
        return
    rank, ws = world()
    cpu_ok = d.get_backend() == "gloo"

    AR = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int)
    AG = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p)

    def allreduce(buf, count, dtype):
        ct = ctypes.c_double if dtype == 0 else ctypes.c_int64
        arr = np.ctypeslib.as_array(ctypes.cast(buf, ctypes.POINTER(ct)), shape=(count,))
        tt = torch.from_numpy(arr)
        if cpu_ok:
            d.all_reduce(tt)
        else:
            g = tt.cuda(); d.all_reduce(g); tt.copy_(g.cpu())

    def allgather(inp, nbytes, out):
        src = np.ctypeslib.as_array(ctypes.cast(inp, ctypes.POINTER(ctypes.c_uint8)), shape=(nbytes,))
        dst = np.ctypeslib.as_array(ctypes.cast(out, ctypes.POINTER(ctypes.c_uint8)), shape=(nbytes * ws,))
        ts = torch.from_numpy(src.copy())
        if cpu_ok:
            outs = [torch.empty(nbytes, dtype=torch.uint8) for _ in range(ws)]
            d.all_gather(outs, ts)
            dst[:] = torch.cat(outs).numpy()
        else:
            outs = [torch.empty(nbytes, dtype=torch.uint8, device="cuda") for _ in range(ws)]
            d.all_gather(outs, ts.cuda())
            dst[:] = torch.cat(outs).cpu().numpy()

    ar, ag = AR(allreduce), AG(allgather)
    _CALLBACKS.extend([ar, ag])
    _safe_call(_lib().FB_NetworkInitWithFunctions(ws, rank, ctypes.cast(ar, ctypes.c_void_p), ctypes.cast(ag, ctypes.c_void_p)))


def free_host_network() -> None:
    from ..basic import _lib, _safe_call

    _safe_call(_lib().FB_NetworkFree())
    _CALLBACKS.clear()
