"""Multi-GPU plumbing: rank bootstrap over ``torch.distributed``, host collective injection for the
CPU learners, and the symmetric-heap handle exchange for the in-kernel NVLink collectives.

Typical use (one process per GPU, started with torchrun)::

    torch.cuda.set_device(local_rank); dist.init_process_group("nccl")
    falcata_b200.parallel.init()
    ds = falcata_b200.Dataset(shard_tensor, label).set_global_rows(offset, total_rows)
    bst = falcata_b200.train({"tree_learner": "data", "device_type": "cuda", ...}, ds)
"""
from . import bootstrap
from .bootstrap import announce_departure, assert_peers_alive, enable_peer_check, free_host_network, init_device_fabric, init_host_network, shutdown_device_fabric, world


def init(heap_bytes: int = 256 << 20, device: bool = True, peer_check: bool = False) -> None:
    """Connect this rank to its peers: host collectives always, the device fabric when CUDA is used.

    torchrun exports OMP_NUM_THREADS=1 to every worker unless the user set it; bin finding at ingest is a
    host loop over features, so in that case each rank takes an equal share of the cores instead."""
    import os

    if os.environ.get("TORCHELASTIC_RUN_ID") and os.environ.get("OMP_NUM_THREADS") == "1" and not os.environ.get("FALCATA_KEEP_OMP_THREADS"):
        from ..basic import set_num_threads

        local_world = max(1, int(os.environ.get("LOCAL_WORLD_SIZE", "1")))
        set_num_threads(max(1, min(32, (os.cpu_count() or 1) // local_world)))
    enable_peer_check(peer_check or bool(os.environ.get("FALCATA_PEER_CHECK")))
    init_host_network()
    if device:
        import torch

        if torch.cuda.is_available():
            init_device_fabric(heap_bytes)


def shutdown() -> None:
    import torch

    if torch.cuda.is_available():
        try:
            shutdown_device_fabric()
        except Exception:
            pass
    free_host_network()


__all__ = ["init", "shutdown", "world", "announce_departure", "assert_peers_alive", "enable_peer_check", "init_host_network", "free_host_network", "init_device_fabric", "shutdown_device_fabric", "bootstrap"]
