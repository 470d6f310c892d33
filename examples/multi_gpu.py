"""Data-parallel training with one process per GPU (or per CPU worker when no GPU is visible).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 examples/multi_gpu.py        # 8 GPUs
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/multi_gpu.py --device cpu

Every rank makes the same synthetic data, keeps its block of consecutive rows and tells the Dataset where that block
sits among all rows; the bins are found on a sample drawn by global row number, so every rank count gives the same bins
and, with quantized gradients, the same model. On GPUs the ranks' kernels exchange histograms and best splits through
peer-mapped memory (NVLink / NVSwitch); on CPUs the host learners use torch.distributed (gloo) for their collectives.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    import torch
    import torch.distributed as dist

    import falcata_b200 as fb
    from falcata_b200 import parallel

    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu", choices=["cuda", "cpu"])
    ap.add_argument("--rows", type=int, default=200_000)
    ap.add_argument("--rounds", type=int, default=20)
    args = ap.parse_args()

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if args.device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl" if args.device == "cuda" else "gloo")
        parallel.init(device=args.device == "cuda")      # symmetric heap between the GPUs / host collectives between the workers

    rng = np.random.default_rng(0)                        # the same data on every rank
    X = rng.normal(size=(args.rows, 16)).astype(np.float32)
    y = (X[:, 0] + X[:, 1] * X[:, 2] + 0.3 * rng.normal(size=args.rows) > 0).astype(np.float32)
    lo, hi = args.rows * rank // world, args.rows * (rank + 1) // world
    local = torch.as_tensor(X[lo:hi], device="cuda") if args.device == "cuda" else X[lo:hi]
    train = fb.Dataset(local, y[lo:hi]).set_global_rows(lo, args.rows)

    params = {"objective": "binary", "num_leaves": 63, "max_bin": 63, "learning_rate": 0.1, "device_type": args.device, "verbosity": -1,
              "quant_mode": "fixedpoint", "quant_bins": 64, "tree_learner": "data" if world > 1 else "serial"}
    booster = fb.train(params, train, args.rounds)
    body = booster.model_to_string().split("\nparameters:")[0]
    acc = float(np.mean((np.asarray(booster.predict(X[:20000])) > 0.5) == (y[:20000] > 0.5)))
    print(f"rank {rank} of {world}: model md5 {hashlib.md5(body.encode()).hexdigest()}, accuracy on 20000 rows {acc:.4f}", flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
