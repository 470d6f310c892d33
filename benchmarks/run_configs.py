"""The five benchmark configurations of the project, on synthetic data of the stated shapes.

    python benchmarks/run_configs.py --config 3 --rounds 20            # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/run_configs.py --config 4 --rounds 20

Config 1 runs the host learner; 2-5 run the device engine (rows sharded over the ranks: tree_learner=data,
voting for config 4). Timing: 3 untimed warm-up rounds, then ``--rounds`` rounds between CUDA events, max over
ranks; the value printed is seconds per 1000 rounds. ``--rows-scale`` shrinks the row count (stated in the
output) for smoke runs. Config 5 also times device prediction of all its rows with the trained model.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _repeat_trees(fb, bst, n_trees):
    """A booster whose forest is the trained trees repeated until there are ``n_trees`` of them (same shapes and
    depths as the trained ones, so traversal cost per tree is that of the real model)."""
    import re

    text = bst.model_to_string()
    head, rest = text.split("\nTree=0\n", 1)
    body, tail = rest.split("\nend of trees\n", 1)
    trees = re.split(r"\nTree=\d+\n", "\n" + "Tree=0\n" + body)
    trees = [t for t in trees if t.strip()]
    if len(trees) >= n_trees:
        return bst
    reps = [trees[i % len(trees)] for i in range(n_trees)]
    sizes = " ".join(str(len(f"Tree={i}\n{t}\n\n")) for i, t in enumerate(reps))
    head = re.sub(r"tree_sizes=.*", "tree_sizes=" + sizes, head)
    model = head + "\n" + "".join(f"Tree={i}\n{t.strip()}\n\n\n" for i, t in enumerate(reps)) + "end of trees\n" + tail
    return fb.Booster(model_str=model)


def reference_arm(args) -> None:
    """The same configuration through the reference's own Python API (`falcata` from baseline/_ref), on one GPU; the data
    generator is loaded by file path so that this repository's package is never imported in the process."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import bench

    ref_dir = os.path.join(root, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref_dir, "falcata", "lib", "lib_falcata.so")):
        print(json.dumps({"config": args.config, "impl": "reference", "unavailable": "baseline/_ref holds no built reference (python baseline/build_reference.py)"}))
        return
    import numpy as np
    import torch

    os.environ.setdefault("NCCL_P2P_DISABLE", "0")
    bench._preload(["libnvrtc.so.12", "libnccl.so.2"])
    sys.path.insert(0, ref_dir)
    try:
        import falcata
    except Exception as e:   # noqa: BLE001
        print(json.dumps({"config": args.config, "impl": "reference", "unavailable": f"the built reference does not load here: {type(e).__name__}: {str(e)[:160]}"}))
        return

    class _Quiet:
        def info(self, msg): pass
        def warning(self, msg): print(msg, file=sys.stderr)
    falcata.register_logger(_Quiet())
    synthetic = bench.load_synthetic()
    group = None
    try:
        if args.config == 1:
            X, y = synthetic.binary_small(device="cpu")
            p = {"objective": "binary", "num_leaves": 31, "max_bin": 255, "learning_rate": 0.1, "device_type": "cpu", "verbosity": -1}
            ds = falcata.Dataset(X.numpy(), y.numpy(), params={"device_type": "cpu", "max_bin": 255, "verbosity": -1}); ds.construct()
            t0 = time.perf_counter()
            bst = falcata.train(p, ds, 100)
            dt = time.perf_counter() - t0
            acc = float(((bst.predict(X.numpy()) > 0.5) == (y.numpy() > 0.5)).mean())
            print(json.dumps({"config": 1, "impl": "reference", "s_per_1000_rounds": dt * 10, "train_accuracy": acc}))
            return
        dev = "cuda:0"
        torch.cuda.set_device(0)
        if args.config == 2:
            total = int(11_000_000 * args.rows_scale)
            X, y = synthetic.binary_higgs_like(total, device=dev)
            p = {"objective": "binary", "num_leaves": 255, "max_bin": 63, "learning_rate": 0.1, "quant_mode": "stochastic", "quant_bins": 4, "max_depth": 8}
        elif args.config == 3:
            total = int(1_000_000 * args.rows_scale)
            X, y = synthetic.regression_wide(total, device=dev)
            p = {"objective": "regression", "num_leaves": 255, "max_bin": 16, "feature_fraction": 0.1, "enable_bundle": True, "quant_mode": "fixedpoint", "quant_bins": 64}
        elif args.config == 4:
            total = int(5_000_000 * args.rows_scale)
            X, y = synthetic.multiclass(total, device=dev)
            p = {"objective": "multiclass", "num_class": 10, "num_leaves": 127, "max_bin": 255, "quant_mode": "none"}
        else:
            totalq = int(100_000 * args.rows_scale)
            X, y, group = synthetic.ranking(totalq, device=dev)
            total = totalq * 100
            p = {"objective": "lambdarank", "metric": "ndcg", "eval_at": "10", "num_leaves": 255}
        p.update({"device_type": "cuda", "verbosity": -1, "tree_learner": "serial", "cuda_precision": "fp32"})
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ds = falcata.Dataset(X, y.cpu().numpy(), group=None if group is None else group.numpy(), params={"max_bin": p.get("max_bin", 255), "device_type": "cuda", "verbosity": -1})
        bst = falcata.Booster(p, ds)
        torch.cuda.synchronize()
        construct_s = time.perf_counter() - t0
        for _ in range(max(3, args.warmup)):
            bst.update()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.rounds):
            bst.update()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        out = {"config": args.config, "impl": "reference", "n_gpus": 1, "rows_total": total, "rounds_timed": args.rounds, "s_per_1000_rounds": dt * 1000.0 / args.rounds,
               "construct_seconds": construct_s, "timing": "wall clock around update() calls with a device synchronize on both sides"}
        try:
            out["train_metric"] = bst.eval_train()
        except Exception as e:   # noqa: BLE001
            out["train_metric"] = f"unavailable: {type(e).__name__}"
        print(json.dumps(out, default=str))
    except Exception as e:   # noqa: BLE001
        print(json.dumps({"config": args.config, "impl": "reference", "unavailable": f"the reference raised on this configuration: {type(e).__name__}: {str(e)[:200]}"}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--rounds", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--rows-scale", type=float, default=1.0)
    ap.add_argument("--plan", default="auto")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"], help="reference: the unmodified reference built under baseline/_ref, one process, one GPU (config 1: its CPU learner)")
    ap.add_argument("--predict-trees", type=int, default=1000, help="config 5: size of the forest that the timed device prediction walks (the trained trees, repeated)")
    ap.add_argument("--grow-policy", default="level", choices=["level", "leaf"], help="level: gain-ranked budget per level; leaf: exact best-first trees")
    args = ap.parse_args()

    if args.impl == "reference":
        reference_arm(args)
        return

    import numpy as np
    import torch

    import falcata_b200 as fb
    from falcata_b200.utils import synthetic

    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0")); local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.config == 1:
        X, y = synthetic.binary_small(device="cpu")
        p = {"objective": "binary", "num_leaves": 31, "max_bin": 255, "learning_rate": 0.1, "device_type": "cpu", "quant_mode": "none", "verbosity": -1}
        ds = fb.Dataset(X.numpy(), y.numpy(), params=p).construct()   # binning is outside the timed region, as in the reference arm
        t0 = time.perf_counter()
        bst = fb.train(p, ds, 100)
        dt = time.perf_counter() - t0
        pr = bst.predict(X.numpy())
        acc = float(((pr > 0.5) == (y.numpy() > 0.5)).mean())
        print(json.dumps({"config": 1, "impl": "ours", "seconds_100_rounds": dt, "s_per_1000_rounds": dt * 10, "train_accuracy": acc,
                          "threads": fb.get_num_threads()}))
        return

    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from falcata_b200 import parallel

        parallel.init(heap_bytes=1 << 30)
    dev = f"cuda:{local}"
    group = None
    extra = {}
    if args.config == 2:
        total = int(11_000_000 * args.rows_scale); off, n = synthetic.shard(total, rank, world)
        X, y = synthetic.binary_higgs_like(n, offset=off, device=dev)
        p = {"objective": "binary", "num_leaves": 255, "max_bin": 63, "learning_rate": 0.1, "quant_mode": "stochastic", "quant_bins": 4}
    elif args.config == 3:
        total = int(1_000_000 * args.rows_scale); off, n = synthetic.shard(total, rank, world)
        X, y = synthetic.regression_wide(n, offset=off, device=dev)
        p = {"objective": "regression", "num_leaves": 255, "max_bin": 16, "feature_fraction": 0.1, "enable_bundle": True, "quant_mode": "fixedpoint", "quant_bins": 64}
    elif args.config == 4:
        total = int(5_000_000 * args.rows_scale); off, n = synthetic.shard(total, rank, world)
        X, y = synthetic.multiclass(n, offset=off, device=dev)
        p = {"objective": "multiclass", "num_class": 10, "num_leaves": 127, "max_bin": 255, "quant_mode": "none", "top_k": 20}
        extra["tree_learner"] = "voting" if world > 1 else "serial"
    else:
        totalq = int(100_000 * args.rows_scale); qoff, nq = synthetic.shard(totalq, rank, world)
        X, y, group = synthetic.ranking(nq, query_offset=qoff, device=dev)
        total = totalq * 100; off, n = qoff * 100, nq * 100
        p = {"objective": "lambdarank", "metric": "ndcg", "eval_at": "10", "num_leaves": 255}
    p.update({"device_type": "cuda", "verbosity": -1, "cuda_plan": args.plan, "grow_policy": args.grow_policy, "tree_learner": extra.get("tree_learner", "data" if world > 1 else "serial")})
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ds = fb.Dataset(X, y.cpu().numpy(), group=None if group is None else group.numpy(), params={"max_bin": p["max_bin"] if "max_bin" in p else 255, "enable_bundle": p.get("enable_bundle", True)})
    ds = ds.set_global_rows(off, total)
    bst = fb.Booster(p, ds)
    torch.cuda.synchronize()
    construct_s = time.perf_counter() - t0
    for _ in range(max(3, args.warmup)):
        bst.update()

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.rounds):
        bst.update()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    out = {"config": args.config, "impl": "ours", "n_gpus": world, "rows_total": total, "rounds_timed": args.rounds, "s_per_1000_rounds": float(ms.item()) / args.rounds,
           "construct_seconds": construct_s, "dataset": ds.info(), "train_metric": bst.eval_train(), "plan": args.plan, "gpu_launches_total": bst.gpu_launches()}
    if args.config == 5:
        # batch inference on the device with a 1000-tree model of the trained trees' shape: the rounds trained so far, repeated
        barrier()
        forest = _repeat_trees(fb, bst, args.predict_trees)
        forest.predict(X[:1000], raw_score=True)          # warm-up (module load, allocator)
        p0 = torch.cuda.Event(enable_timing=True); p1 = torch.cuda.Event(enable_timing=True)
        p0.record()
        pred = forest.predict(X, raw_score=True)           # includes packing the forest and its upload
        p1.record(); torch.cuda.synchronize()
        out["predict_rows"] = int(X.shape[0]); out["predict_trees"] = forest.num_trees(); out["predict_ms"] = p0.elapsed_time(p1)
        out["predict_trained_trees"] = bst.num_trees()
        out["predict_ns_per_row_tree"] = 1e6 * p0.elapsed_time(p1) / (X.shape[0] * max(1, forest.num_trees()))
        host = forest.predict(X[:2000].cpu().numpy(), raw_score=True)
        out["predict_max_abs_diff_vs_host_2000_rows"] = float(np.abs(np.asarray(host) - pred[:2000].cpu().numpy()).max())
        del pred
    if rank == 0:
        print(json.dumps(out, default=str))
    if world > 1:
        import torch.distributed as dist
        from falcata_b200 import parallel

        parallel.shutdown(); dist.destroy_process_group()


if __name__ == "__main__":
    main()
