"""Shared-GPU guard: wait until the GPU is quiet enough to measure on, or say that it is busy.

    python tests/gates/gpu_guard.py [--min-free-gb 8] [--max-util 20] [--sustain 15] [--timeout 600]

Exit codes: 0 = quiet for ``--sustain`` seconds, 3 = still busy at the timeout, 4 = no GPU / no nvidia-smi.
Only reads ``nvidia-smi`` queries; it changes nothing on the GPU.
Parity: tests/gates/gpu_guard.py:L37-72 of the reference (>= 8 GB free and <= 20 % utilisation sustained 15 s).
"""
from __future__ import annotations

import argparse
import subprocess
import sys
import time
from typing import Callable, List, Optional, Tuple

Sample = Tuple[float, float]   # (free GiB, utilisation %)


def query(index: int = 0, run: Callable[..., str] = None) -> Optional[Sample]:
    run = run or (lambda cmd: subprocess.run(cmd, capture_output=True, text=True, timeout=20).stdout)
    try:
        out = run(["nvidia-smi", f"--id={index}", "--query-gpu=memory.free,utilization.gpu", "--format=csv,noheader,nounits"])
        free_mib, util = [x.strip() for x in out.strip().splitlines()[0].split(",")]
        return float(free_mib) / 1024.0, float(util)
    except Exception:
        return None


def foreign_processes(own_pids: List[int], index: int = 0, run: Callable[..., str] = None) -> List[int]:
    """PIDs of compute processes on the GPU that are not ours."""
    run = run or (lambda cmd: subprocess.run(cmd, capture_output=True, text=True, timeout=20).stdout)
    try:
        out = run(["nvidia-smi", f"--id={index}", "--query-compute-apps=pid", "--format=csv,noheader"])
    except Exception:
        return []
    pids = [int(x) for x in out.split() if x.strip().isdigit()]
    return [p for p in pids if p not in own_pids]


def wait_quiet(min_free_gb: float, max_util: float, sustain: float, timeout: float, sampler: Callable[[], Optional[Sample]] = query,
               sleep: Callable[[float], None] = time.sleep, clock: Callable[[], float] = time.monotonic, period: float = 1.0) -> int:
    start = clock(); quiet_since = None
    while True:
        s = sampler()
        if s is None:
            return 4
        now = clock()
        if s[0] >= min_free_gb and s[1] <= max_util:
            quiet_since = quiet_since if quiet_since is not None else now
            if now - quiet_since >= sustain:
                return 0
        else:
            quiet_since = None
        if now - start >= timeout:
            return 3
        sleep(period)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpu", type=int, default=0); ap.add_argument("--min-free-gb", type=float, default=8.0); ap.add_argument("--max-util", type=float, default=20.0)
    ap.add_argument("--sustain", type=float, default=15.0); ap.add_argument("--timeout", type=float, default=600.0)
    a = ap.parse_args()
    rc = wait_quiet(a.min_free_gb, a.max_util, a.sustain, a.timeout, sampler=lambda: query(a.gpu))
    print({0: "GPU quiet", 3: "GPU busy", 4: "no GPU visible"}[rc])
    return rc


if __name__ == "__main__":
    sys.exit(main())
