"""Leave-one-out ablation over the planner's switches on the binary benchmark shape.

Every ``cuda_plan`` switch that does not change the model is flipped on its own against the planner's defaults; each
arm trains ``--warmup`` untimed and ``--rounds`` timed boosting rounds on the same device-resident dataset (CUDA events
around the timed rounds) and reports milliseconds per round, the ratio to the default plan and the md5 of the model
text (equal for every arm: the switches choose between implementations of the same arithmetic). One JSON line per arm
goes to ``--out`` (JSONL) and to stdout.

    python benchmarks/ablation.py --rows 11000000 --rounds 10 --out ablation.jsonl

Parity: benchmarks/ablation.py of the reference (leave-one-out over its plan keys, JSONL).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=11_000_000)
    ap.add_argument("--rounds", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--grow-policy", default="level", choices=["level", "leaf"])
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    import torch

    import falcata_b200 as fb
    from falcata_b200 import tuner
    from falcata_b200.utils import synthetic

    X, y = synthetic.binary_higgs_like(args.rows, seed=0, device="cuda")
    ds = fb.Dataset(X, y.cpu().numpy(), params={"max_bin": 63}).construct()
    del X
    base = {"objective": "binary", "num_leaves": 255, "max_bin": 63, "learning_rate": 0.1, "quant_mode": "stochastic", "quant_bins": 4, "device_type": "cuda",
            "verbosity": -1, "min_data_in_leaf": 20, "grow_policy": args.grow_policy}

    def run(plan: str):
        bst = fb.Booster(dict(base, cuda_plan=plan), ds)
        for _ in range(args.warmup):
            bst.update()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.rounds):
            bst.update()
        e1.record(); torch.cuda.synchronize()
        md5 = hashlib.md5(bst.model_to_string().split("\nparameters:")[0].encode()).hexdigest()
        return e0.elapsed_time(e1) / args.rounds, md5

    sink = open(args.out, "w") if args.out else None
    base_ms, base_md5 = run("auto")
    rows = [{"plan": "auto", "ms_per_round": base_ms, "ratio_to_default": 1.0, "model_md5": base_md5}]
    for key in tuner.TUNABLE:
        flips = dict(tuner._DEFAULT_ON); flips[key] = not flips[key]
        plan = tuner.plan_string(flips)
        try:
            ms, md5 = run(plan)
            rows.append({"plan": plan, "ms_per_round": ms, "ratio_to_default": ms / base_ms, "model_md5": md5, "same_model": md5 == base_md5})
        except Exception as e:   # a switch that does not apply to this shape
            rows.append({"plan": plan, "error": str(e)[:200]})
    for r in rows:
        r.update({"rows": args.rows, "rounds": args.rounds, "warmup": args.warmup, "grow_policy": args.grow_policy})
        line = json.dumps(r)
        print(line)
        if sink:
            sink.write(line + "\n")
    if sink:
        sink.close()


if __name__ == "__main__":
    main()
