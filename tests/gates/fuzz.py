"""Randomised parity gate: random training specifications, each trained on the device and on the host learner.

Per specification (`sample_spec`): data shape and type (float / small integers, missing values, zero-heavy columns,
categorical columns), objective (regression / binary / multiclass), quantization mode and level count, tree shape,
row and column sampling, bin count and a random subset of `cuda_plan` flips. Checks (`check_spec`):

* the device run finishes and its model survives a text round trip;
* quantized device training is deterministic: a second run gives the same model md5;
* the device metric is not much worse than the host learner's on the same data (the two may differ in sampling
  streams and summation order, so a tolerance applies; coarse stochastic quantization gets a wider one);
* on a machine without a GPU the device arm is the host learner with quantization and the reference arm is the
  host learner without: still a check of the quantized path against the exact one.

    python tests/gates/fuzz.py --specs 20 --seed 1            # exit 1 when a specification fails
    python tests/gates/fuzz.py --replay '<json spec>'

Idea after tests/gates/fuzz.py of the reference; the specification space and the code are this repository's own.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
METRIC_TOLERANCE = 0.12        # relative, device against host
COARSE_TOLERANCE = 0.35        # stochastic rounding with few levels on small leaves is noisy by design

PLAN_KEYS = ["device_controller:off", "fused_tail:off", "fused_scan:off", "hist_lane:off", "hist_lane_red:off", "col_major_part:off", "compact_view:off",
             "pack4:off", "bulk_root:off", "gh_in_row:on"]


def sample_spec(rng):
    objective = str(rng.choice(["regression", "binary", "multiclass"]))
    quant_mode = str(rng.choice(["stochastic", "stochastic", "fixedpoint", "none"]))
    ncat = int(rng.choice([0, 0, 0, 1, 3]))
    spec = {
        "rows": int(rng.choice([1500, 4000, 12000, 30000])), "cols": int(rng.choice([4, 12, 40, 150])),
        "dtype": str(rng.choice(["float32", "float64", "small_int"])), "nan_frac": float(rng.choice([0.0, 0.0, 0.1, 0.35])),
        "zero_frac": float(rng.choice([0.0, 0.0, 0.75])), "cat_cards": [int(c) for c in rng.choice([5, 18, 60, 200], size=ncat)],
        "objective": objective, "num_class": int(rng.integers(3, 7)) if objective == "multiclass" else 1,
        "quant_mode": quant_mode, "quant_bins": int(rng.choice([0, 4, 16, 256])) if quant_mode != "none" else 0,
        "num_leaves": int(rng.choice([4, 15, 63, 255])), "max_depth": int(rng.choice([-1, -1, 3, 6, 10])),
        "min_data_in_leaf": int(rng.choice([1, 5, 20, 80])), "learning_rate": float(rng.choice([0.3, 0.1, 0.02])),
        "feature_fraction": float(rng.choice([1.0, 1.0, 0.5, 0.2])), "bagging_fraction": float(rng.choice([1.0, 1.0, 0.6])),
        "max_bin": int(rng.choice([7, 15, 63, 255])), "grow_policy": str(rng.choice(["level", "level", "leaf"])),
        "lambda_l2": float(rng.choice([0.0, 1.0, 10.0])), "rounds": int(rng.choice([5, 15, 40])), "seed": int(rng.integers(0, 2 ** 31 - 1)),
        "plan": ["auto"] + [k for k in PLAN_KEYS if rng.random() < 0.15],
    }
    # keep the host arm cheap: the product of all sizes is bounded by trimming rounds first, then rows
    cost = lambda s: s["rows"] * s["cols"] * s["rounds"] * s["num_class"]
    while cost(spec) > 2.5e8 and spec["rounds"] > 5:
        spec["rounds"] = max(5, spec["rounds"] // 2)
    while cost(spec) > 2.5e8 and spec["rows"] > 1500:
        spec["rows"] = max(1500, spec["rows"] // 2)
    return spec


def make_data(spec):
    import numpy as np

    rng = np.random.default_rng(spec["seed"])
    n, f = spec["rows"], spec["cols"]
    if spec["dtype"] == "small_int":
        X = rng.integers(-6, 8, size=(n, f)).astype(np.float64)
    else:
        X = rng.normal(size=(n, f)).astype(np.float64)
    w = rng.normal(size=f) * (rng.random(size=f) < 0.5)
    cats = []
    for j, card in enumerate(spec["cat_cards"]):
        if j >= f:
            break
        X[:, j] = rng.integers(0, card, size=n); cats.append(j)
        w[j] = 0.0
    signal = X @ w + 0.5 * X[:, -1] * X[:, f // 2]
    for j in cats:
        signal = signal + np.where(X[:, j].astype(int) % 2 == 0, 0.8, -0.8)
    signal = signal / (np.std(signal) + 1e-9)
    if spec["zero_frac"] > 0:
        mask = rng.random(size=X.shape) < spec["zero_frac"]; mask[:, cats] = False
        X[mask] = 0.0
    if spec["nan_frac"] > 0:
        mask = rng.random(size=X.shape) < spec["nan_frac"]; mask[:, cats] = False
        X[mask] = np.nan
    if spec["objective"] == "regression":
        y = signal + 0.3 * rng.normal(size=n)
    elif spec["objective"] == "binary":
        y = (signal + 0.5 * rng.normal(size=n) > 0).astype(np.float64)
    else:
        k = spec["num_class"]
        y = np.clip(np.digitize(signal + 0.4 * rng.normal(size=n), np.quantile(signal, np.linspace(0, 1, k + 1)[1:-1])), 0, k - 1).astype(np.float64)
    if spec["dtype"] == "float32":
        X = X.astype(np.float32)
    return X, y, cats


def run(spec, device, exact=False):
    """Train `spec` on `device`; returns {md5, metric, higher_better, trees} or {error}."""
    import numpy as np

    sys.path.insert(0, str(ROOT))
    import falcata_b200 as fb

    try:
        X, y, cats = make_data(spec)
        metric = {"regression": "l2", "binary": "binary_logloss", "multiclass": "multi_logloss"}[spec["objective"]]
        p = {"objective": spec["objective"], "num_leaves": spec["num_leaves"], "max_depth": spec["max_depth"], "min_data_in_leaf": spec["min_data_in_leaf"],
             "learning_rate": spec["learning_rate"], "feature_fraction": spec["feature_fraction"], "bagging_fraction": spec["bagging_fraction"],
             "bagging_freq": 1 if spec["bagging_fraction"] < 1.0 else 0, "max_bin": spec["max_bin"], "lambda_l2": spec["lambda_l2"], "grow_policy": spec["grow_policy"],
             "quant_mode": "none" if exact else spec["quant_mode"], "metric": metric, "verbosity": -1, "device_type": device, "seed": 3, "min_data_per_group": 10}
        if spec["quant_bins"] and not exact and spec["quant_mode"] != "none":
            p["quant_bins"] = spec["quant_bins"]
        if spec["objective"] == "multiclass":
            p["num_class"] = spec["num_class"]
        if device == "cuda":
            p["cuda_plan"] = ",".join(spec["plan"])
        rec = {}
        ds = fb.Dataset(X, y, categorical_feature=cats if cats else "auto", params={"max_bin": spec["max_bin"]})
        bst = fb.train(p, ds, spec["rounds"], valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(rec)])
        text = bst.model_to_string()
        pred = np.asarray(bst.predict(X))
        if not np.all(np.isfinite(pred)):
            return {"error": "non-finite predictions"}
        if not np.array_equal(pred, np.asarray(fb.Booster(model_str=text).predict(X))):
            return {"error": "predictions change after a text round trip"}
        return {"md5": hashlib.md5(text.split("\nparameters:")[0].encode()).hexdigest(), "metric": float(rec["train"][metric][-1]), "higher_better": False,
                "trees": bst.num_trees()}
    except Exception as e:
        return {"error": f"{type(e).__name__}: {str(e)[:300]}"}


def check_spec(spec, device):
    """Returns (failures, notes)."""
    fails, notes = [], []
    a = run(spec, device)
    if "error" in a:
        return [f"{device} run failed: {a['error']}"], notes
    if spec["quant_mode"] != "none":
        b = run(spec, device)
        if "error" in b:
            fails.append(f"{device} rerun failed: {b['error']}")
        elif a["md5"] != b["md5"]:
            fails.append(f"{device} training is not deterministic: {a['md5']} != {b['md5']}")
    # reference arm: the host learner; exact gradients when the arm under test is the host learner itself
    c = run(spec, "cpu", exact=(device == "cpu"))
    if "error" in c:
        fails.append(f"host run failed: {c['error']}")
        return fails, notes
    coarse = spec["quant_mode"] == "stochastic" and (spec["quant_bins"] in (0, 4)) and spec["min_data_in_leaf"] < 20
    tol = COARSE_TOLERANCE if coarse else METRIC_TOLERANCE
    ref, cur = c["metric"], a["metric"]
    if cur > ref + abs(ref) * tol + 1e-6:
        (notes if coarse and cur <= ref + abs(ref) * 1.0 else fails).append(f"{device} metric {cur:.6f} against host {ref:.6f} (tolerance {tol})")
    return fails, notes


def main(argv=None) -> int:
    import numpy as np

    ap = argparse.ArgumentParser()
    ap.add_argument("--specs", type=int, default=10); ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default=None, choices=["cpu", "cuda"]); ap.add_argument("--replay", default=None); ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    sys.path.insert(0, str(ROOT))
    import falcata_b200 as fb

    device = args.device or ("cuda" if fb.cuda_available() else "cpu")
    rng = np.random.default_rng(args.seed)
    specs = [json.loads(args.replay)] if args.replay else [sample_spec(rng) for _ in range(args.specs)]
    bad = 0; log = []
    for i, spec in enumerate(specs):
        fails, notes = check_spec(spec, device)
        log.append({"spec": spec, "failures": fails, "notes": notes})
        print(f"[{i}] {'FAIL' if fails else 'ok  '} {spec['objective']:10s} {spec['quant_mode']:10s} rows={spec['rows']} cols={spec['cols']} leaves={spec['num_leaves']} "
              f"{'; '.join(fails + notes)}", flush=True)
        if fails:
            bad += 1
            print("     replay:", json.dumps(spec))
    if args.out:
        Path(args.out).write_text(json.dumps({"device": device, "log": log}, indent=1))
    print(f"{len(specs)} specifications, {bad} failed, device kind {device}")
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
