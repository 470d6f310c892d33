"""Worker of the multi-GPU tests: trains on this rank's shard of a seeded synthetic data set and has
rank 0 write the model text. Run directly (1 rank) or under torch.distributed.run (N ranks)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=200000)
    ap.add_argument("--rounds", type=int, default=5)
    ap.add_argument("--leaves", type=int, default=31)
    ap.add_argument("--quant", default="stochastic")
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-spins", type=int, default=0)
    ap.add_argument("--skip-rank", type=int, default=-1, help="this rank leaves before training (failure-detection test)")
    args = ap.parse_args()
    import torch

    import falcata_b200 as fb
    from falcata_b200 import parallel
    from falcata_b200.utils import synthetic

    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        parallel.init()
    off, n = synthetic.shard(args.rows, rank, world)
    X, y = synthetic.binary_higgs_like(n, offset=off, seed=1, device=f"cuda:{local}")
    params = {"objective": "binary", "num_leaves": args.leaves, "max_bin": 63, "quant_mode": args.quant, "tree_learner": "data" if world > 1 else "serial",
              "device_type": "cuda", "verbosity": -1, "min_data_in_leaf": 20, "metric": "binary_logloss"}
    ds = fb.Dataset(X, y.cpu().numpy(), params={"max_bin": 63}).set_global_rows(off, args.rows)
    bst = fb.Booster(params, ds)
    for _ in range(args.rounds):
        bst.update()
    ll = bst.eval_train()[0][2]
    if rank == 0:
        with open(args.out, "w") as f:
            f.write(bst.model_to_string(num_iteration=-1).split("\nparameters:")[0])
        print(f"world={world} logloss={ll:.6f}")
    if world > 1:
        import torch.distributed as dist

        parallel.shutdown()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
