"""One rank of the CPU multi-process tests (gloo). Started by test_cpu_distributed.py.

Modes:
  train   every rank trains on its row shard (data / voting) or on all rows (feature) and rank 0 writes
          the model text
  fail    rank 1 raises before its first collective; the other ranks must come back with an error from
          the bounded process-group timeout instead of waiting for ever
"""
import argparse
import datetime
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="train")
    ap.add_argument("--learner", default="data")
    ap.add_argument("--quant", default="none")
    ap.add_argument("--rows", type=int, default=6000)
    ap.add_argument("--rounds", type=int, default=10)
    ap.add_argument("--out", default="")
    ap.add_argument("--device", default="cpu", help="cpu: host learners; cuda: the device engine, one GPU per rank (gloo is still the plumbing)")
    ap.add_argument("--top-k", type=int, default=12)
    ap.add_argument("--leaves", type=int, default=15)
    args = ap.parse_args()

    import torch.distributed as dist

    import falcata_b200 as fb
    from falcata_b200 import parallel
    from util import make_binary

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=8 if args.mode == "fail" else 120))
    if args.mode == "fail" and rank == 1:
        # a rank that dies on the host before joining any collective
        raise SystemExit(7)
    if args.device == "cuda":
        import torch

        torch.cuda.set_device(rank)
    parallel.init(device=args.device == "cuda")
    X, y = make_binary(args.rows, 12)
    params = {"objective": "binary", "num_leaves": args.leaves, "max_bin": 63, "verbosity": -1, "device_type": args.device, "tree_learner": args.learner,
              "grow_policy": "level", "quant_mode": args.quant, "min_data_in_leaf": 5, "seed": 5}
    if args.learner == "voting":
        params["top_k"] = args.top_k   # 12 = all features voted in: must equal the data-parallel result
    try:
        if args.learner == "feature":
            ds = fb.Dataset(X, y).set_global_rows(0, args.rows)       # every rank holds all rows
        else:
            lo, hi = args.rows * rank // world, args.rows * (rank + 1) // world
            ds = fb.Dataset(X[lo:hi], y[lo:hi]).set_global_rows(lo, args.rows)
        bst = fb.train(params, ds, args.rounds)
    except Exception as e:  # the failure test expects to land here on the surviving ranks
        print("TRAIN_ERROR", type(e).__name__, str(e)[:200], flush=True)
        raise SystemExit(3)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            f.write(bst.model_to_string())
    parallel.shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
