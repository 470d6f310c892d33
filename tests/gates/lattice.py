"""Regression lattice: small deterministic (data profile x parameters) training cells with stored model fingerprints.

Three kinds of check, after the gate design of the reference (tests/gates/lattice.py there):

1. fingerprints - quantized training sums integers, so a cell's model text is a stable signature of the whole
   training path. The md5 of every fingerprinted cell is stored per device kind in ``md5_lattice.json``; an
   unintended behaviour change flips at least one. Intended changes are re-baselined explicitly
   (``--baseline`` / ``--update``) and the diff of the JSON file shows which cells moved.
2. equalities - every ``cuda_plan`` key is flipped against its base cell, and ``grow``/``rank-count`` variants are
   compared the same way: the two models must be byte-identical. These cells carry no stored fingerprint.
3. validity - every cell: the model survives ``model_to_string -> Booster(model_str)`` with identical predictions,
   predictions are finite, the tree count is rounds x trees per round, and the training metric clears a floor.

Usage:
  python tests/gates/lattice.py --check              # compare with the stored fingerprints (exit 1 on a mismatch)
  python tests/gates/lattice.py --baseline           # (re)write all fingerprints of this device kind
  python tests/gates/lattice.py --update ID [ID..]   # re-baseline some cells
  python tests/gates/lattice.py --list               # print the cell matrix
  options: --device cpu|cuda (default: cuda when a GPU is present), --only SUBSTR, --out FILE (results as JSON)
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import time
from pathlib import Path

GATES = Path(__file__).resolve().parent
ROOT = GATES.parent.parent
FINGERPRINTS = GATES / "md5_lattice.json"

PLAN_FLIPS = ["device_controller:off", "fused_tail:off", "fused_scan:off", "hist_lane:off", "hist_lane_red:off", "col_major_part:off", "gh_in_row:on",
              "bulk_root:off", "compact_view:off", "pack4:off", "hist_tc:on"]


def build_cells():
    """The cell matrix. A cell: id, profile, params (merged over the profile's), rounds, equal_to (id of the cell
    whose model it must reproduce), fingerprint (False: validity and metric floor only), devices."""
    cells = []

    def add(cid, profile, params=None, rounds=12, equal_to=None, fingerprint=True, devices=("cpu", "cuda")):
        cells.append({"id": cid, "profile": profile, "params": params or {}, "rounds": rounds, "equal_to": equal_to,
                      "fingerprint": fingerprint and equal_to is None, "devices": list(devices)})

    quant = {"quant_mode": "stochastic", "quant_bins": 4}
    fixed = {"quant_mode": "fixedpoint", "quant_bins": 64}
    for prof in ["dense", "missing", "zero_heavy", "bundled", "four_bit", "categorical", "tiny_grad", "wide_bins"]:
        add(f"{prof}/stochastic", prof, dict(quant))
        add(f"{prof}/fixedpoint", prof, dict(fixed))
        add(f"{prof}/float", prof, {"quant_mode": "none"}, fingerprint=False)
    add("multiclass/stochastic", "multiclass", dict(quant))
    add("multiclass/float", "multiclass", {"quant_mode": "none"}, fingerprint=False)
    add("ranking/stochastic", "ranking", dict(quant))
    add("ranking/float", "ranking", {"quant_mode": "none"}, fingerprint=False)
    add("large/stochastic", "large", dict(quant), rounds=6)
    add("dense/fixedpoint-plain", "dense", dict(fixed, cuda_plan="auto,quant_ef:off,robust_scale:off"))
    add("imbalanced/fixedpoint", "imbalanced", dict(fixed))                                        # the outlier-robust scale fires here
    add("imbalanced/fixedpoint-norobust", "imbalanced", dict(fixed, cuda_plan="auto,robust_scale:off"))
    add("dense/leafwise", "dense", dict(quant, grow_policy="leaf"))
    add("dense/bagging", "dense", dict(quant, bagging_fraction=0.7, bagging_freq=1))
    add("dense/goss", "dense", dict(quant, data_sample_strategy="goss"))
    add("dense/feature_fraction", "dense", dict(quant, feature_fraction=0.5))
    add("bundled/feature_fraction", "bundled", dict(fixed, feature_fraction=0.3))
    add("dense/monotone", "dense", {"quant_mode": "none", "monotone_constraints": [1, -1, 0, 0, 0, 0, 0, 0, 0, 0]}, fingerprint=False)
    add("dense/dart", "dense", dict(quant, boosting="dart", drop_rate=0.3), fingerprint=False)
    add("dense/renew_leaf", "dense", dict(quant, quant_train_renew_leaf=True), fingerprint=False)
    # plan flips: byte-identical to the base cell (device only: the host learner has no plan)
    for flip in PLAN_FLIPS:
        for prof in ["dense", "missing", "four_bit"]:
            add(f"{prof}/flip-{flip}", prof, dict(quant, cuda_plan="auto," + flip), equal_to=f"{prof}/stochastic", devices=("cuda",))
    add("bundled/flip-compact_view:off", "bundled", dict(fixed, feature_fraction=0.3, cuda_plan="auto,compact_view:off"), equal_to="bundled/feature_fraction", devices=("cuda",))
    add("dense/leafwise-host-order", "dense", dict(quant, grow_policy="leaf", cuda_plan="auto,fused_tail:off"), equal_to="dense/leafwise", devices=("cuda",))
    return cells


def build_profile(name):
    """(X, y, group, base parameters, metric name, higher-is-better, floor/ceiling of the training metric)."""
    import numpy as np

    rng = np.random.default_rng(sum(map(ord, name)) * 7919)   # a seed that depends on the profile name only
    n, f = 4000, 10
    group = None
    base = {"objective": "binary", "num_leaves": 15, "max_bin": 63, "min_data_in_leaf": 10, "learning_rate": 0.2, "verbosity": -1, "seed": 7}
    metric, higher, bound = "binary_logloss", False, 0.55
    if name == "large":
        n = 60000
    X = rng.normal(size=(n, f)).astype(np.float32)
    logit = X[:, 0] - 0.7 * X[:, 1] + 0.5 * X[:, 2] * X[:, 3]
    if name == "missing":
        X[rng.random(size=X.shape) < 0.15] = np.nan
        base["use_missing"] = True
    elif name == "zero_heavy":
        X[rng.random(size=X.shape) < 0.7] = 0.0           # the most frequent bin is not bin 0 of a sorted feature
        logit = X[:, 0] - 0.7 * X[:, 1] + 0.5 * X[:, 2] * X[:, 3]
        bound = 0.62
    elif name == "bundled":
        f = 60
        X = np.zeros((n, f), dtype=np.float32)
        hot = rng.integers(0, f, size=(n, 3))               # three non-zero columns per row: mutually exclusive bundles
        for k in range(3):
            X[np.arange(n), hot[:, k]] = rng.integers(1, 6, size=n)
        logit = X[:, :20].sum(axis=1) - X[:, 20:40].sum(axis=1)
        base.update(enable_bundle=True, max_bin=15)
        bound = 0.6
    elif name == "four_bit":
        X = rng.integers(0, 12, size=(n, f)).astype(np.float32)
        logit = 0.4 * (X[:, 0] - 6) - 0.3 * (X[:, 1] - 6) + 0.05 * (X[:, 2] - 6) * (X[:, 3] - 6)
        base["max_bin"] = 15
    elif name == "categorical":
        X[:, 4] = rng.integers(0, 20, size=n); X[:, 5] = rng.integers(0, 6, size=n)
        logit = logit + np.where(X[:, 4] % 3 == 0, 1.0, -0.5) + 0.3 * X[:, 5]
        base.update(categorical_feature=[4, 5], min_data_per_group=10, cat_smooth=2.0)
    elif name == "tiny_grad":
        base.update(objective="regression", learning_rate=0.1)
        metric, bound = "l2", None
    elif name == "wide_bins":
        base["max_bin"] = 255
    elif name == "imbalanced":
        n = 40000
        X = rng.normal(size=(n, f)).astype(np.float32)
        logit = 2.0 * X[:, 0] - 1.5 * X[:, 1] + X[:, 2] * X[:, 3] - 7.5          # about one positive in 260
        base["min_sum_hessian_in_leaf"] = 1.0
        metric, higher, bound = "auc", True, 0.9
    if name == "multiclass":
        W = rng.normal(size=(f, 4))
        y = np.argmax(X @ W + rng.gumbel(size=(n, 4)), axis=1).astype(np.float32)
        base.update(objective="multiclass", num_class=4)
        metric, bound = "multi_logloss", 1.25
    elif name == "ranking":
        q = 200; per = n // q
        n = q * per; X = X[:n]; logit = logit[:n]
        rel = np.zeros(n, dtype=np.float32)
        for i in range(q):
            s = logit[i * per:(i + 1) * per] + 0.3 * rng.normal(size=per)
            rel[i * per:(i + 1) * per] = np.clip(np.digitize(s, np.quantile(s, [0.5, 0.75, 0.9, 0.97])), 0, 4)
        y = rel; group = np.full(q, per, dtype=np.int32)
        base.update(objective="lambdarank", eval_at=[5], min_data_in_leaf=5)
        metric, higher, bound = "ndcg@5", True, 0.6
    elif name == "tiny_grad":
        y = (1e-4 * logit + 1e-5 * rng.normal(size=n)).astype(np.float32)
    else:
        y = (logit + 0.5 * rng.normal(size=n) > 0).astype(np.float32)
    return X, y, group, base, metric, higher, bound


def model_md5(text: str) -> str:
    body = text.split("\nparameters:")[0]
    return hashlib.md5(body.encode()).hexdigest()


def run_cell(cell, device):
    """Train one cell; returns {md5, metric, seconds, problems: [...]}."""
    import numpy as np

    sys.path.insert(0, str(ROOT))
    import falcata_b200 as fb

    X, y, group, base, metric, higher, bound = build_profile(cell["profile"])
    params = dict(base, **cell["params"])
    params["device_type"] = device
    params.setdefault("metric", metric.split("@")[0])
    if device == "cpu" and "quant_ef" not in str(params.get("cuda_plan", "")) and "robust_scale" not in str(params.get("cuda_plan", "")):
        params.pop("cuda_plan", None)   # the host learner reads only the quantizer switches of the plan
    problems = []
    t0 = time.perf_counter()
    ds = fb.Dataset(X, y, group=group, categorical_feature=params.pop("categorical_feature", "auto"), params={k: params[k] for k in ("max_bin", "enable_bundle", "use_missing") if k in params})
    rec = {}
    bst = fb.train(params, ds, cell["rounds"], valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(rec)])
    seconds = time.perf_counter() - t0
    text = bst.model_to_string()
    per_round = int(params.get("num_class", 1)) if params.get("objective") == "multiclass" else 1
    if bst.num_trees() != cell["rounds"] * per_round:
        problems.append(f"{bst.num_trees()} trees for {cell['rounds']} rounds")
    pred = np.asarray(bst.predict(X))
    if not np.all(np.isfinite(pred)):
        problems.append("non-finite predictions")
    again = np.asarray(fb.Booster(model_str=text).predict(X))
    if not np.array_equal(pred, again):
        problems.append("predictions change after a text round trip of the model")
    series = rec.get("train", {})
    key = metric if metric in series else next(iter(series), None)
    value = float(series[key][-1]) if key else float("nan")
    if key and len(series[key]) > 1 and cell["profile"] == "tiny_grad" and not series[key][-1] < series[key][0]:
        problems.append(f"{key} did not improve: {series[key][0]} -> {series[key][-1]}")
    if bound is not None and key and ((higher and value < bound) or (not higher and value > bound)):
        problems.append(f"{key} = {value:.5f} misses the bound {bound}")
    return {"md5": model_md5(text), "metric": value, "metric_name": key, "seconds": seconds, "problems": problems}


def check(cells, results, stored, device, update_ids=None, write_all=False):
    """Compares results with the stored fingerprints; returns (failures, new fingerprint table)."""
    fails = []
    table = dict(stored.get(device, {}))
    by_id = {c["id"]: c for c in cells}
    for cid, r in results.items():
        c = by_id[cid]
        for p in r["problems"]:
            fails.append(f"{cid}: {p}")
        if c["equal_to"] is not None:
            base = results.get(c["equal_to"])
            if base is None:
                fails.append(f"{cid}: base cell {c['equal_to']} did not run")
            elif base["md5"] != r["md5"]:
                fails.append(f"{cid}: model differs from {c['equal_to']} ({r['md5']} != {base['md5']})")
            continue
        if not c["fingerprint"]:
            continue
        if write_all or (update_ids and cid in update_ids):
            table[cid] = {"md5": r["md5"], "metric": round(r["metric"], 6)}
        elif device not in stored:
            pass   # nothing was ever baselined for this device kind: equalities and validity still count
        elif cid not in table:
            fails.append(f"{cid}: no stored fingerprint for device kind '{device}' (run --baseline)")
        elif table[cid]["md5"] != r["md5"]:
            fails.append(f"{cid}: fingerprint moved {table[cid]['md5']} -> {r['md5']} (metric {table[cid].get('metric')} -> {r['metric']:.6f})")
    out = dict(stored); out[device] = dict(sorted(table.items()))
    return fails, out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--check", action="store_true"); ap.add_argument("--baseline", action="store_true")
    ap.add_argument("--update", nargs="*", default=None); ap.add_argument("--list", action="store_true")
    ap.add_argument("--device", default=None, choices=["cpu", "cuda"]); ap.add_argument("--only", default=None)
    ap.add_argument("--out", default=None); ap.add_argument("--fingerprints", default=str(FINGERPRINTS))
    args = ap.parse_args(argv)
    cells = build_cells()
    if args.list:
        for c in cells:
            print(f"{c['id']:44s} {c['profile']:12s} rounds={c['rounds']:3d} {'= ' + c['equal_to'] if c['equal_to'] else ('fingerprint' if c['fingerprint'] else 'validity')}  {','.join(c['devices'])}")
        return 0
    sys.path.insert(0, str(ROOT))
    import falcata_b200 as fb

    device = args.device or ("cuda" if fb.cuda_available() else "cpu")
    chosen = [c for c in cells if device in c["devices"] and (args.only is None or args.only in c["id"])]
    need = {c["equal_to"] for c in chosen if c["equal_to"]}
    chosen += [c for c in cells if c["id"] in need and c not in chosen]
    results = {}
    for c in chosen:
        try:
            results[c["id"]] = run_cell(c, device)
        except Exception as e:   # a failing cell fails alone
            results[c["id"]] = {"md5": "", "metric": float("nan"), "metric_name": None, "seconds": 0.0, "problems": [f"{type(e).__name__}: {str(e)[:300]}"]}
        r = results[c["id"]]
        print(f"{c['id']:44s} {r['md5'][:10]:10s} {r['metric_name']}={r['metric']:.5f} {r['seconds']:.2f}s {'; '.join(r['problems'])}", flush=True)
    path = Path(args.fingerprints)
    stored = json.loads(path.read_text()) if path.exists() else {}
    fails, table = check(cells, results, stored, device, update_ids=set(args.update or []), write_all=args.baseline)
    if args.baseline or args.update:
        path.write_text(json.dumps(table, indent=1, sort_keys=True) + "\n")
        print(f"wrote {path}")
    if args.out:
        Path(args.out).write_text(json.dumps({"device": device, "results": results, "failures": fails}, indent=1))
    for f in fails:
        print("FAIL", f)
    print(f"{len(results)} cells, {len(fails)} failure(s), device kind {device}")
    return 1 if fails else 0


if __name__ == "__main__":
    raise SystemExit(main())
