"""A/B of the root-level histogram construct: lane kernel (SIMT, warp-private tiles) against the tcgen05 one-hot
instance (`cuda_plan=hist_tc:on`), inside real training rounds.

Each arm trains a few rounds of the binary benchmark shape in a child process with per-stage CUDA-event spans dumped
(`FALCATA_STAGE_TIMING=1 FALCATA_STAGE_DUMP=1`); the first "histogram" span of every tree is the root level (all rows,
in order), which is the only level the tensor-core instance covers. Prints the median root span per arm, the useful
bytes per second (rows x (32 bin bytes + 4 gradient bytes)) and the fraction of the measured copy bandwidth.

Usage: python benchmarks/hist_tc_ab.py [--rows 6000000] [--rounds 12]
"""
import argparse
import json
import os
import re
import statistics
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

CHILD = r"""
import sys, os
sys.path.insert(0, {root!r})
import torch
import falcata_b200 as fb
from falcata_b200.utils import synthetic
X, y = synthetic.binary_higgs_like({rows}, seed=0, device="cuda")
ds = fb.Dataset(X, y.cpu().numpy(), params={{"max_bin": 63}})
p = {{"objective": "binary", "num_leaves": 255, "max_bin": 63, "quant_mode": "stochastic", "quant_bins": 4, "device_type": "cuda", "verbosity": -1,
     "min_data_in_leaf": 20, "cuda_plan": {plan!r}}}
bst = fb.Booster(p, ds)
for _ in range({rounds}):
    bst.update()
torch.cuda.synchronize()
print("MODEL_MD5", __import__("hashlib").md5(bst.model_to_string().split("\nparameters:")[0].encode()).hexdigest())
"""


def run(plan: str, rows: int, rounds: int):
    env = dict(os.environ, FALCATA_STAGE_TIMING="1", FALCATA_STAGE_DUMP="1")
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT, rows=rows, plan=plan, rounds=rounds)], capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise SystemExit(r.stderr[-2000:])
    spans, roots = [], []
    prev = None
    for line in r.stderr.splitlines():
        m = re.match(r"\[stage\] (\S+) ([0-9.]+) us", line)
        if not m:
            continue
        name, us = m.group(1), float(m.group(2))
        if name == "histogram" and prev == "quantize+root":
            roots.append(us)
        prev = name
    md5 = [l.split()[1] for l in r.stdout.splitlines() if l.startswith("MODEL_MD5")]
    return roots[3:], md5[0] if md5 else None   # the first trees warm up


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=6_000_000)
    ap.add_argument("--rounds", type=int, default=12)
    args = ap.parse_args()
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    out = {}
    for name, plan in (("lane (SIMT)", "auto"), ("tcgen05 one-hot", "auto,hist_tc:on")):
        roots, md5 = run(plan, args.rows, args.rounds)
        med = statistics.median(roots)
        gbs = args.rows * 36 / (med * 1e-6) / 1e9
        out[name] = {"root_span_us_median": med, "useful_GB_per_s": gbs, "fraction_of_measured_copy_bandwidth": gbs / hbm, "spans": len(roots), "model_md5": md5}
    print(json.dumps({"rows": args.rows, "groups": 28, "bins_per_group": 63, "hbm_gbs_reference": hbm, "arms": out}, indent=1))


if __name__ == "__main__":
    main()
