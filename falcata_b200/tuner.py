"""Plan tuner with a wisdom file.

Every ``cuda_plan`` switch except the quantizer ones chooses between implementations that produce the same model, so
they can be chosen by the clock. ``tune`` times a few boosting rounds of the actual training job per candidate plan
(coordinate descent over the switches: flip one, keep the flip if it is faster by more than the noise margin), returns
the fastest plan and remembers it in a small JSON "wisdom" file keyed by the workload's shape and the device, so that
the next training of the same shape on the same kind of GPU starts from the known-best plan:

    plan = fb.tuner.tune(params, train_set)                 # probes, stores, returns e.g. "auto,fused_scan:off"
    fb.train({**params, "cuda_plan": "wisdom"}, train_set)  # looks the plan up (``auto`` when nothing is stored)

Parity: src/treelearner/cuda/cuda_single_gpu_tree_learner.cpp:L3069-3243 (tier-one tuner probing knob values during
training, wisdom keyed by shape and device, FFTW-wisdom style). Differences by design: the knobs here are the planner's
switches rather than numeric block-shape floors (block shapes were fixed from sweeps on B200), and the probe runs as
an explicit call before training instead of inside the first rounds.
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional

# switches whose two settings give byte-identical models (the quantizer switches robust_scale / quant_ef change the model)
TUNABLE = ["hist_lane_red", "fused_tail", "fused_scan", "col_major_part", "bulk_root", "gh_in_row", "compact_view", "pack4", "hist_float_red"]
_DEFAULT_ON = {"hist_lane_red": True, "fused_tail": True, "fused_scan": True, "col_major_part": True, "bulk_root": True, "gh_in_row": False, "compact_view": True,
               "pack4": True, "hist_float_red": False}


def wisdom_path() -> Path:
    p = os.environ.get("FALCATA_WISDOM")
    return Path(p) if p else Path(os.environ.get("HOME", "/tmp")) / ".cache" / "falcata_b200" / "wisdom.json"


def _device_name() -> str:
    try:
        import torch

        if torch.cuda.is_available():
            return torch.cuda.get_device_name(torch.cuda.current_device()).replace(" ", "_")
    except Exception:
        pass
    return "cpu"


def wisdom_key(params: Dict[str, Any], num_data: int, num_features: int, world: int = 1, device: Optional[str] = None) -> str:
    """Workload signature: rows (rounded to a quarter octave, so that a few more rows reuse the entry), features, tree
    shape, quantization, ranks and the device name."""
    import math

    rows_bucket = int(round(4 * math.log2(max(1, num_data))))
    return "v1:{}:{}:{}:{}:{}:{}:{}:{}:{}".format(rows_bucket, num_features, params.get("num_leaves", 31), params.get("max_depth", -1), params.get("max_bin", 255),
                                                  params.get("quant_mode", "auto"), params.get("quant_bins", 0), world, device or _device_name())


def plan_string(flips: Dict[str, bool]) -> str:
    parts = ["auto"] + [f"{k}:{'on' if v else 'off'}" for k, v in sorted(flips.items()) if v != _DEFAULT_ON[k]]
    return ",".join(parts)


def load_wisdom(path: Optional[Path] = None) -> Dict[str, Any]:
    path = path or wisdom_path()
    try:
        return json.loads(Path(path).read_text())
    except Exception:
        return {}


def lookup(params: Dict[str, Any], num_data: int, num_features: int, world: int = 1, path: Optional[Path] = None) -> str:
    """The stored plan for this workload, or ``auto``."""
    entry = load_wisdom(path).get(wisdom_key(params, num_data, num_features, world))
    return entry["plan"] if isinstance(entry, dict) and "plan" in entry else "auto"


def _store(key: str, entry: Dict[str, Any], path: Optional[Path]) -> None:
    path = Path(path or wisdom_path())
    table = load_wisdom(path)
    table[key] = entry
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(".tmp")
    tmp.write_text(json.dumps(table, indent=1, sort_keys=True))
    tmp.replace(path)


def _time_plan(params: Dict[str, Any], train_set: Any, plan: str, rounds: int, warmup: int) -> float:
    """Milliseconds per boosting round of `plan` on the device (CUDA events; wall clock without a GPU)."""
    from .basic import Booster, cuda_available

    bst = Booster(dict(params, cuda_plan=plan, verbosity=-1), train_set)
    for _ in range(warmup):
        bst.update()
    if cuda_available():
        import torch

        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(rounds):
            bst.update()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / rounds
    t0 = time.perf_counter()
    for _ in range(rounds):
        bst.update()
    return (time.perf_counter() - t0) * 1000.0 / rounds


def tune(params: Dict[str, Any], train_set: Any, rounds: int = 8, warmup: int = 3, margin: float = 0.02, switches: Optional[List[str]] = None,
         path: Optional[Path] = None, timer: Optional[Callable[[str], float]] = None, store: bool = True) -> str:
    """Probe the plan switches on this training job and return the fastest plan string.

    One coordinate-descent pass: starting from the planner's defaults, each switch is flipped in turn and the flip is kept
    when it is faster than the current best by more than ``margin`` (relative). ``timer(plan) -> ms per round`` replaces
    the built-in measurement (tests, external harnesses). The result is stored under the workload's key."""
    from .basic import Dataset

    if not isinstance(train_set, Dataset):
        raise TypeError("tune() takes the training Dataset")
    measure = timer or (lambda plan: _time_plan(params, train_set, plan, rounds, warmup))
    flips = dict(_DEFAULT_ON)
    best_plan = plan_string(flips)
    best_ms = measure(best_plan)
    trail = [{"plan": best_plan, "ms": best_ms}]
    for key in (switches or TUNABLE):
        trial = dict(flips); trial[key] = not trial[key]
        plan = plan_string(trial)
        try:
            ms = measure(plan)
        except Exception as e:   # a switch that does not apply to this workload is skipped
            trail.append({"plan": plan, "error": str(e)[:120]})
            continue
        trail.append({"plan": plan, "ms": ms})
        if ms < best_ms * (1.0 - margin):
            flips, best_plan, best_ms = trial, plan, ms
    if store:
        try:
            train_set.construct()
            nd, nf = train_set.num_data(), train_set.num_feature()
        except Exception:
            nd, nf = 0, 0
        from .parallel import bootstrap

        _store(wisdom_key(params, nd, nf, bootstrap.world()[1]), {"plan": best_plan, "ms_per_round": best_ms, "probes": trail, "when": time.strftime("%Y-%m-%d %H:%M:%S")}, path)
    return best_plan
