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
    ap.add_argument("--learner", default="data", help="data: rows sharded; feature: rows replicated, features split")
    ap.add_argument("--top-k", type=int, default=20)
    ap.add_argument("--categorical", action="store_true", help="treat the last two columns (rounded) as categorical")
    ap.add_argument("--grow-policy", default="level")
    ap.add_argument("--plan", default="auto", help="cuda_plan string")
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
        parallel.init(peer_check=args.skip_rank >= 0)
    replicated = args.learner == "feature" and world > 1
    off, n = (0, args.rows) if replicated else synthetic.shard(args.rows, rank, world)
    X, y = synthetic.binary_higgs_like(n, offset=off, seed=1, device=f"cuda:{local}")
    cat = None
    if args.categorical:
        X[:, -2:] = torch.clamp(torch.round(X[:, -2:] * 4) + 12, 0, 30)
        cat = [X.shape[1] - 2, X.shape[1] - 1]
    if args.max_spins > 0:
        from falcata_b200.basic import _lib

        _lib().FB_FabricSetMaxSpins(int(args.max_spins))
    params = {"objective": "binary", "num_leaves": args.leaves, "max_bin": 63, "quant_mode": args.quant, "grow_policy": args.grow_policy, "tree_learner": args.learner if world > 1 else "serial",
              "device_type": "cuda", "verbosity": -1, "min_data_in_leaf": 20, "metric": "binary_logloss", "top_k": args.top_k, "cuda_plan": args.plan}
    ds = fb.Dataset(X, y.cpu().numpy(), params={"max_bin": 63}, categorical_feature=cat if cat else "auto")
    ds = ds.set_replicated() if replicated else ds.set_global_rows(off, args.rows)
    try:
        bst = fb.Booster(params, ds)
        for _ in range(2):
            bst.update()
        if world > 1 and args.skip_rank >= 0:
            # One rank leaves between rounds with nothing of its own in flight. It says so on the host
            # first; the barrier orders that notice before every other rank's next liveness check, so the
            # others stop BEFORE their next launch.
            import time
            import torch.distributed as dist

            torch.cuda.synchronize()
            if rank == args.skip_rank:
                parallel.announce_departure("test")
            dist.barrier()
            if rank == args.skip_rank:
                print(f"rank {rank} leaves after round 2", flush=True)
                time.sleep(3.0)   # stay mapped while the others notice and stop
                os._exit(0)
        for _ in range(max(0, args.rounds - 2)):
            bst.update()
    except Exception as e:
        print("TRAIN_ERROR", str(e)[:300], flush=True)
        os._exit(5)
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
