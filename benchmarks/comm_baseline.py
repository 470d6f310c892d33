"""What the library-call baseline costs: NCCL collectives on the message shapes of one boosting level.

The fused kernels of the engine move, per level, the histogram slices of the level's smaller children
(tasks x total_bins x 8 bytes, reduce-scatter) and one best-split record per child (all-gather). This script
times the NCCL calls a non-fused implementation would issue for the same shapes - all-reduce (what the reference
does), reduce-scatter and all-gather - with CUDA events, max over ranks, after warm-up.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/comm_baseline.py
"""
import json
import os

import torch
import torch.distributed as dist


def timed(fn, iters=50, warmup=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(); dist.barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1000.0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world, rank = dist.get_world_size(), dist.get_rank()
    total_bins = 28 * 64                      # config 2: 28 feature groups of 64 bins
    rows = []
    for level in range(8):
        tasks = 1 << level                    # smaller children constructed at this level
        n = tasks * total_bins                # packed 64-bit bins
        n = (n + world - 1) // world * world
        hist = torch.zeros(n, dtype=torch.int64, device="cuda")
        out = torch.zeros(n // world, dtype=torch.int64, device="cuda")
        rec = torch.zeros(2 * tasks * 40, dtype=torch.int32, device="cuda")            # one 160-byte record per child
        gathered = torch.zeros(world * rec.numel(), dtype=torch.int32, device="cuda")
        rows.append({"level": level + 1, "tasks": tasks, "hist_bytes": n * 8,
                     "allreduce_us": timed(lambda: dist.all_reduce(hist)),
                     "reduce_scatter_us": timed(lambda: dist.reduce_scatter_tensor(out, hist)),
                     "allgather_best_us": timed(lambda: dist.all_gather_into_tensor(gathered, rec))})
    if rank == 0:
        tot_ar = sum(r["allreduce_us"] for r in rows); tot_rs = sum(r["reduce_scatter_us"] + r["allgather_best_us"] for r in rows)
        print(json.dumps({"n_gpus": world, "per_level": rows, "per_tree_allreduce_only_us": tot_ar, "per_tree_reduce_scatter_plus_allgather_us": tot_rs}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
