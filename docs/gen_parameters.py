"""Writes docs/Parameters.md from the parameter table of the native core (csrc/include/fb/config.h).

    python docs/gen_parameters.py            # rewrite the file
    python docs/gen_parameters.py --check    # exit 1 when the file is out of date (used by the tests)

The table in config.h is the single source: name, type, default and aliases of every parameter. Notes on what a
parameter does on this framework's device engine are kept in NOTES below.
"""
from __future__ import annotations

import os
import re
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CONFIG_H = os.path.join(ROOT, "falcata_b200", "csrc", "include", "fb", "config.h")
OUT = os.path.join(ROOT, "docs", "Parameters.md")

NOTES = {
    "device_type": "`cuda` (default when a GPU is visible): the device engine; `cpu`: the host learner",
    "grow_policy": "`level` (default): whole levels per launch batch, gain-ranked when the leaf budget binds; `leaf`: exact best-first trees (device: num_leaves <= 512)",
    "quant_mode": "`none`, `stochastic` (Philox rounding keyed on the global row id), `fixedpoint` (robust scale + error feedback); `auto` follows `use_quantized_grad`",
    "quant_bins": "gradient levels; 0 = automatic (raised for small leaves on large data, lowered to keep 32-bit histograms exact)",
    "cuda_plan": "`auto[,key:on|off]*` or `wisdom` (the plan stored by `falcata_b200.tuner.tune`)",
    "tree_learner": "`serial`, `data`, `feature`, `voting`; on GPUs the collectives run inside the kernels over peer memory, on CPUs over the injected or TCP network",
    "monotone_constraints_method": "`basic` (host and device), `intermediate` and `advanced` (host learner; a device booster hands training to it)",
    "forcedsplits_filename": "host learner and, on one GPU, the device engine",
    "linear_tree": "host learner; on one GPU without row sampling the trees grow on the device and the leaf regressions are solved on the host",
    "boosting": "`gbdt`, `dart`, `rf` (all three on the device engine), `goss` as `data_sample_strategy`",
    "histogram_pool_size": "MB of cached leaf histograms in the host learner (least recently used dropped); the device engine keeps all",
    "num_machines": "with `machines` / `machine_list_filename` and `local_listen_port`: distributed CPU training over TCP",
    "max_bin": "device engine: up to 255 (one byte per feature group); larger values train on the host learner",
}


def parse():
    text = open(CONFIG_H).read()
    rows = []
    for m in re.finditer(r'^\s*X\(([^,]+),\s*([a-z_0-9]+),\s*(.*?),\s*"([^"]*)"\)\s*\\?\s*$', text, re.M):
        ctype, name, default, aliases = m.group(1).strip(), m.group(2), m.group(3).strip(), m.group(4)
        kind = {"std::string": "string", "double": "float", "int": "int", "bool": "bool", "int64_t": "int"}.get(ctype, ctype)
        rows.append((name, kind, default.strip('"') if kind == "string" else default, aliases))
    return rows


def render(rows):
    out = ["# Parameters", "",
           "Generated from `falcata_b200/csrc/include/fb/config.h` by `python docs/gen_parameters.py`; do not edit by hand.",
           "Every parameter can be given under any of its aliases, in a Python `dict`, in a command-line config file or as `key=value`.", "",
           f"{len(rows)} parameters.", "",
           "| parameter | type | default | aliases | notes |", "|---|---|---|---|---|"]
    for name, kind, default, aliases in rows:
        shown = f"`{default}`" if default != "" else "(empty)"
        out.append(f"| `{name}` | {kind} | {shown} | {', '.join('`' + a + '`' for a in aliases.split(',') if a)} | {NOTES.get(name, '')} |")
    return "\n".join(out) + "\n"


def main() -> int:
    doc = render(parse())
    if "--check" in sys.argv:
        current = open(OUT).read() if os.path.exists(OUT) else ""
        if current != doc:
            print("docs/Parameters.md is out of date: run python docs/gen_parameters.py", file=sys.stderr)
            return 1
        return 0
    with open(OUT, "w") as f:
        f.write(doc)
    print("wrote", OUT)
    return 0


if __name__ == "__main__":
    sys.exit(main())
