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


def _bernoulli_rows(t: Any, n: int, offset: int, seed: int, p: float) -> Any:
    """Local indices of the rows picked for the bin sample: a draw keyed on (seed, GLOBAL row id), made by the
    library on the device for CUDA tensors and on the host otherwise - the same rows either way."""
    import torch

    from ..basic import _lib

    lib = _lib()
    cnt = ctypes.c_int(0)
    # the draw needs the row ids only, not the data: with a GPU at hand it runs there even for a host matrix
    on_gpu = t.is_cuda or (torch.cuda.is_available() and n >= (1 << 20))
    if on_gpu:
        gdev = t.device if t.is_cuda else torch.device("cuda", torch.cuda.current_device())
        out = torch.empty(max(1, n), dtype=torch.int32, device=gdev)
        with torch.cuda.device(gdev):
            torch.cuda.current_stream().synchronize()
            rc = lib.FB_OpBernoulliRowsDevice(ctypes.c_int(n), ctypes.c_longlong(offset), ctypes.c_uint(seed & 0xFFFFFFFF), ctypes.c_double(p),
                                              ctypes.c_void_p(out.data_ptr()), ctypes.byref(cnt))
    else:
        out = torch.empty(max(1, n), dtype=torch.int32)
        rc = lib.FB_OpBernoulliRowsHost(ctypes.c_int(n), ctypes.c_longlong(offset), ctypes.c_uint(seed & 0xFFFFFFFF), ctypes.c_double(p),
                                        ctypes.c_void_p(out.data_ptr()), ctypes.byref(cnt))
    if rc != 0:
        lib.FB_OpsLastError.restype = ctypes.c_char_p
        raise RuntimeError(lib.FB_OpsLastError().decode())
    return out[: cnt.value].to(t.device).long()


def gather_bin_sample(t: Any, sample_cnt: int, seed: int, offset: int = 0, total: int = 0, replicated: bool = False,
                      after_draw: Any = None) -> Tuple[np.ndarray, int]:
    """Rows used to find bin boundaries.

    A global row is sampled iff a Philox number keyed on (seed, global row id) is below ``sample_cnt / total``. The choice depends only on the GLOBAL
    row id, so the sample - and with it every bin boundary - is the same however the rows are sharded
    over ranks. Each rank contributes the sampled rows of its shard; the shards are concatenated in
    rank order. ``replicated``: every rank holds ALL rows (feature-parallel training), so the local sample
    is already the global one and nothing is exchanged. ``after_draw``: called once the row draw (which may run on the
    device) and, with several ranks, the exchange of the sample are done and only host work remains. Returns (sample [ns, ncol] in the matrix's own element
    type - float16/32/64, int8/16/32, uint8 - so nothing is widened on the way to the host; total rows)."""
    import torch

    rank, ws = world()
    n = t.shape[0]
    d = None if replicated else _dist()
    if replicated:
        rank, ws, offset, total = 0, 1, 0, n
    if total <= 0:
        total = n
        if d and ws > 1:
            cnt = torch.tensor([n], dtype=torch.int64, device=(t.device if t.is_cuda else torch.device("cuda", torch.cuda.current_device())) if d.get_backend() == "nccl" else "cpu")
            d.all_reduce(cnt)
            total = int(cnt.item())
            offs = [None] * ws
            d.all_gather_object(offs, n)
            offset = int(sum(offs[:rank]))
    p = min(1.0, sample_cnt / max(1, total))
    idx = _bernoulli_rows(t, n, offset, seed, p)
    exchange = bool(d and ws > 1)
    if after_draw is not None and not exchange:
        after_draw()
    keep = t.dtype in (torch.float16, torch.float32, torch.float64, torch.int8, torch.int16, torch.int32, torch.uint8)
    sdt = t.dtype if keep else torch.float64
    picked = t[idx].to(sdt)
    if d and ws > 1:
        # tensor collectives (no pickling): sizes first, then the rows padded to the largest shard
        on_dev = d.get_backend() == "nccl"   # NCCL moves device tensors only: a host sample rides through the current device
        cdev = (picked.device if picked.is_cuda else torch.device("cuda", torch.cuda.current_device())) if on_dev else torch.device("cpu")
        sizes = torch.zeros(ws, dtype=torch.int64, device=cdev)
        sizes[rank] = picked.shape[0]
        d.all_reduce(sizes)
        sizes = sizes.cpu().tolist()
        cap = max(1, max(sizes))
        padded = torch.zeros((cap, t.shape[1]), dtype=sdt, device=cdev)
        padded[: picked.shape[0]] = picked.to(cdev)
        outs = torch.empty((ws, cap, t.shape[1]), dtype=sdt, device=cdev)
        d.all_gather_into_tensor(outs, padded) if on_dev else d.all_gather(list(outs.unbind(0)), padded)
        outs = outs.cpu().numpy()
        if after_draw is not None:
            after_draw()   # the sample's small copies are through: the caller's large copy no longer delays them
        local = np.concatenate([outs[r, : sizes[r]] for r in range(ws)], axis=0)
    else:
        local = picked.cpu().numpy()
    if local.shape[0] == 0:
        local = t[:1].to(sdt).cpu().numpy()
    return local, total


# ---- liveness on the host ---------------------------------------------------------------------
# A rank that stops (an exception in user code, a planned departure) announces it in the process
# group's key-value store; with the check enabled every rank looks for such notices before it enqueues
# the next boosting round, so nobody launches kernels that would wait for a peer that is gone. Ranks
# that vanish without notice are caught by the bounded flag waits of the kernels (status word).
_PEER_CHECK = False


def _store():
    from torch.distributed import distributed_c10d as c10d

    return c10d._get_default_store()


def enable_peer_check(on: bool = True) -> None:
    global _PEER_CHECK
    _PEER_CHECK = bool(on)


def peer_check_enabled() -> bool:
    return _PEER_CHECK and _dist() is not None


def announce_departure(reason: str = "left") -> None:
    """Tell the other ranks that this rank will not take part in further rounds."""
    d = _dist()
    if d is None:
        return
    _store().set(f"falcata/left/{d.get_rank()}", reason)
    _store().add("falcata/left_count", 1)


def assert_peers_alive() -> None:
    """Raise if some rank has announced its departure (one small store read)."""
    d = _dist()
    if d is None:
        return
    if _store().add("falcata/left_count", 0) > 0:
        gone = [r for r in range(d.get_world_size()) if _store().check([f"falcata/left/{r}"])]
        raise RuntimeError(f"rank(s) {gone} left the job: stopping before the next launch")


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


def init_device_fabric(heap_bytes: int = 256 << 20) -> None:
    """Allocate this rank's symmetric heap on the current CUDA device and map every peer's heap.

    The heap holds the histogram pool slices, the split-candidate slots, the per-split row counts and
    the flag words that the training kernels read and write on peer GPUs directly over NVLink."""
    import torch

    from ..basic import _lib

    d = _dist()
    if d is None or d.get_world_size() == 1:
        return
    rank, ws = world()
    lib = _lib()
    lib.FB_FabricLastError.restype = ctypes.c_char_p
    buf = ctypes.create_string_buffer(64)
    if lib.FB_FabricCreate(rank, ws, ctypes.c_int64(heap_bytes), buf) != 0:
        raise RuntimeError(lib.FB_FabricLastError().decode())
    mine = torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8)
    dev = torch.device("cuda", torch.cuda.current_device()) if d.get_backend() == "nccl" else torch.device("cpu")
    outs = [torch.empty(64, dtype=torch.uint8, device=dev) for _ in range(ws)]
    d.all_gather(outs, mine.to(dev))
    handles = b"".join(bytes(o.cpu().numpy().tobytes()) for o in outs)
    if lib.FB_FabricConnect(handles) != 0:
        raise RuntimeError(lib.FB_FabricLastError().decode())
    d.barrier()


def shutdown_device_fabric() -> None:
    from ..basic import _lib

    d = _dist()
    if d is not None:
        import torch

        torch.cuda.synchronize()
        d.barrier()
    _lib().FB_FabricDestroy()
