"""Headline benchmark: seconds per 1000 boosting rounds on the 11M x 28 binary configuration.

Config (the second of the project's five benchmark configurations): 11,000,000 rows x 28 fp32 features (21 N(0,1) + 7 |x_i x_j|), label ~
Bernoulli(sigmoid(x.w + 0.5 x0 x1)); objective=binary, num_leaves=255, max_bin=63, learning_rate=0.1,
quant_mode=stochastic with 4 bins, tree_learner=data, rows sharded over the GPUs of one box.

A "step" is one boosting round: gradients, quantization, every level of tree growth (partition,
histogram construction with its reduce-scatter, split search) and the score update. Steps are timed
on the device with CUDA events, max over ranks. The per-step working set (binned rows, 32 B/row)
is larger than L2, so no explicit L2 flush is needed between steps.

Usage: python bench.py [--gpus N] [--steps K] [--warmup W] [--rows R] [--impl ours|reference]
For N > 1 launch with torchrun (one rank per GPU); RANK / LOCAL_RANK / WORLD_SIZE come from the env.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

ROWS = 11_000_000
PARAMS = {"objective": "binary", "num_leaves": 255, "max_bin": 63, "learning_rate": 0.1, "quant_mode": "stochastic", "quant_bins": 4,
          "cuda_precision": "fp32", "tree_learner": "data", "device_type": "cuda", "verbosity": -1, "min_data_in_leaf": 20, "metric": "binary_logloss"}


class ClockSampler:
    """nvidia-smi SM clock / throttle-reason samples taken while the timed region runs."""

    def __init__(self, index: int) -> None:
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(float(parts[0])); self.max_mhz = float(parts[1])
                    for name, val in zip(names, parts[2:6]):
                        if val.lower().startswith("active"):
                            self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set(); self._t.join(timeout=6)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def reference_arm(args) -> None:
    # The reference needs its external_libs submodules (Eigen, fast_double_parser, fmt); the mounted tree
    # ships them as empty directories and the image has no copy, so it cannot be built offline here.
    ok = os.path.isdir(os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "falcata"))
    if not ok:
        print(json.dumps({"impl": "reference", "unavailable": "reference cannot be built offline: its source tree is not pip-installable (no pyproject at its root) and its external_libs submodules (eigen, fast_double_parser, fmt) are empty and absent from the image"}))
        return
    print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref exists but the native library was never built (missing Eigen / fast_double_parser sources)"}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--rows", type=int, default=ROWS)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--stage-timing", action="store_true")
    ap.add_argument("--plan", default="auto", help="cuda_plan string, e.g. auto,hist_lane:off")
    ap.add_argument("--grow-policy", default=None, choices=["level", "leaf"], help="level: gain-ranked leaf budget per level; leaf: exact best-first trees")
    args = ap.parse_args()
    PARAMS["cuda_plan"] = args.plan
    if args.grow_policy is not None:
        PARAMS["grow_policy"] = args.grow_policy
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.stage_timing:
        os.environ["FALCATA_STAGE_TIMING"] = "1"

    import numpy as np
    import torch

    import falcata_b200 as fb
    from falcata_b200.parallel import bootstrap
    from falcata_b200.utils import synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        from falcata_b200 import parallel

        parallel.init()
    else:
        torch.cuda.set_device(0)
    dev = torch.device("cuda", local_rank)
    warmup = max(3, args.warmup)
    K = args.steps

    off, n_local = synthetic.shard(args.rows, rank, world)
    X, y = synthetic.binary_higgs_like(n_local, offset=off, seed=0, device=str(dev))
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed steps (data already on the device) ----
    ds = fb.Dataset(X, y.cpu().numpy(), params={"max_bin": PARAMS["max_bin"]}).set_global_rows(off, args.rows)
    bst = fb.Booster(PARAMS, ds)
    for _ in range(warmup):
        bst.update()
    barrier()
    l0 = bst.gpu_launches()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        barrier()
        e0.record()
        for _ in range(K):
            bst.update()
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    launches = bst.gpu_launches() - l0
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / K
    stage = bst.stage_report() if args.stage_timing else ""
    logloss = bst.eval_train()[0][2] if bst.eval_train() else None
    del bst, ds

    # ---- end to end through the public API: pinned host matrix -> H2D -> on-device binning -> K rounds,
    # reading the training metric back to the host every round ----
    e2e = None
    if not args.no_e2e:
        Xh = torch.empty(X.shape, dtype=X.dtype, pin_memory=True); Xh.copy_(X)
        yh = y.cpu().numpy()
        del X
        torch.cuda.empty_cache()
        barrier()
        if os.environ.get("FALCATA_TIME_TAG"):
            fb.set_time_tag(True)
        t0 = time.perf_counter()
        # the pinned host matrix goes straight into the public API: the library copies it to the device on a side stream
        # while the host finds the bin boundaries, then bins on the device
        ds2 = fb.Dataset(Xh, yh, params={"max_bin": PARAMS["max_bin"], "device_type": "cuda"}).set_global_rows(off, args.rows)
        b2 = fb.train(dict(PARAMS, is_provide_training_metric=True), ds2, K, valid_sets=[ds2], valid_names=["train"], keep_training_booster=True,
                      callbacks=[fb.record_evaluation({})])
        barrier()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], dtype=torch.float64, device=dev)
        if world > 1:
            import torch.distributed as dist

            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        if os.environ.get("FALCATA_TIME_TAG") and rank == 0:
            print(fb.time_tag_report(), file=sys.stderr)
        e2e = {"value": float(tt.item()) / K * 1000.0, "unit": "s/1000 rounds (ingest from pinned host memory + K rounds + per-round metric read, wall clock / K)",
               "h2d_bytes_per_step": int((Xh.numel() * Xh.element_size() + yh.nbytes) / K), "d2h_bytes_per_step": 16}

    if rank == 0:
        out = {"metric": "s/1000 rounds (device-timed, max over ranks)", "value": ms_per_step, "unit": "s/1000 rounds", "n_gpus": world, "steps": K, "warmup": warmup,
               "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "int16-quantized gradients / fp32 scores (reference: same)",
               "data": "synthetic", "impl": "ours",
               "config": {"model": "gbdt binary 11Mx28, num_leaves=255, max_bin=63, quant_mode=stochastic(4 bins)", "grow_policy": PARAMS.get("grow_policy", "level"), "global_batch": args.rows, "seq_len": 28,
                          "parallelism": f"dp{world}" if world > 1 else "single", "l2": "inputs_larger_than_L2", "train_logloss_after_run": logloss},
               "clocks": clk.summary(), "gpu_launches": int(launches)}
        if e2e is not None:
            out["e2e"] = e2e
        if stage:
            out["stage_ms"] = stage
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist
        from falcata_b200 import parallel

        parallel.shutdown()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
