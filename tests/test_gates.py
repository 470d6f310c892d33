"""The measurement gates on fake inputs (no GPU needed): quiet-GPU guard and the rolling-median perf gate."""
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "gates"))
import gpu_guard  # noqa: E402
import perf_gate  # noqa: E402


def _fake_time():
    t = {"now": 0.0}
    return (lambda: t["now"]), (lambda dt: t.__setitem__("now", t["now"] + dt))


def test_gpu_guard_waits_for_a_sustained_quiet_window():
    clock, sleep = _fake_time()
    samples = iter([(4.0, 90.0)] * 5 + [(60.0, 5.0)] * 3 + [(60.0, 70.0)] + [(60.0, 3.0)] * 40)
    assert gpu_guard.wait_quiet(8, 20, 15, 600, sampler=lambda: next(samples), sleep=sleep, clock=clock) == 0
    assert clock() >= 9 + 15           # the short quiet spell before the burst did not count
    clock, sleep = _fake_time()
    assert gpu_guard.wait_quiet(8, 20, 15, 30, sampler=lambda: (2.0, 99.0), sleep=sleep, clock=clock) == 3
    assert gpu_guard.wait_quiet(8, 20, 15, 30, sampler=lambda: None) == 4
    assert gpu_guard.query(run=lambda cmd: "81234, 7\n") == (81234 / 1024.0, 7.0)
    assert gpu_guard.foreign_processes([11], run=lambda cmd: "11\n4242\n") == [4242]


def test_perf_gate_uses_the_rolling_median_and_needs_two_bad_runs(tmp_path):
    hist = tmp_path / "h.jsonl"
    line = lambda v, **kw: {"value": v, "higher_is_better": False, "clocks": {"reasons": []}, **kw}
    assert perf_gate.gate("k", line(3.0), hist)["status"] == "first"
    for v in (3.05, 2.95, 3.0):
        assert perf_gate.gate("k", line(v), hist)["status"] == "ok"
    assert perf_gate.gate("k", line(3.5), hist)["status"] == "warn"            # +17 %
    # +40 %: flagged, re-measured best of three, still slow -> flag; the next slow run fails
    reruns = iter([line(4.3), line(4.25)])
    assert perf_gate.gate("k", line(4.2), hist, rerun=lambda: next(reruns))["status"] == "flag"
    assert perf_gate.gate("k", line(4.2), hist)["status"] == "fail"
    # a noisy first try that re-measures fine is accepted
    reruns = iter([line(3.02), line(3.4)])
    assert perf_gate.gate("k2", line(3.0), hist)["status"] == "first"
    assert perf_gate.gate("k2", line(4.5), hist, rerun=lambda: next(reruns))["status"] == "ok"
    # contention is not judged and not recorded
    n = len(hist.read_text().splitlines())
    assert perf_gate.gate("k", line(9.9), hist, foreign=[4242])["status"] == "contended"
    assert perf_gate.gate("k", line(9.9, clocks={"reasons": ["hw_thermal_slowdown"]}), hist)["status"] == "contended"
    assert len(hist.read_text().splitlines()) == n
    rows = [json.loads(l) for l in hist.read_text().splitlines()]
    assert [r["accepted"] for r in rows if r["key"] == "k"][-2:] == [False, False]


def test_lattice_cells_match_their_stored_fingerprints_on_the_host_learner():
    """A slice of the regression lattice on the host learner: stored md5 fingerprints of the quantized cells,
    validity checks of all of them. The full matrix (with the plan-flip equalities) runs on the GPU box."""
    import lattice  # noqa: E402

    rc = lattice.main(["--check", "--device", "cpu", "--only", "dense/"])
    assert rc == 0
    rc = lattice.main(["--check", "--device", "cpu", "--only", "/fixedpoint"])
    assert rc == 0


def test_lattice_reports_a_moved_fingerprint(tmp_path):
    import lattice  # noqa: E402

    stored = json.loads(lattice.FINGERPRINTS.read_text())
    stored["cpu"]["dense/stochastic"]["md5"] = "0" * 32
    fp = tmp_path / "fp.json"; fp.write_text(json.dumps(stored))
    assert lattice.main(["--check", "--device", "cpu", "--only", "dense/stochastic", "--fingerprints", str(fp)]) == 1
    cells = {c["id"]: c for c in lattice.build_cells()}
    assert cells["dense/flip-fused_tail:off"]["equal_to"] == "dense/stochastic" and not cells["dense/flip-fused_tail:off"]["fingerprint"]
    assert all(k.split(":")[0] in {"device_controller", "fused_tail", "fused_scan", "hist_lane", "hist_lane_red", "col_major_part", "gh_in_row", "bulk_root",
                                   "compact_view", "pack4", "hist_tc"} for k in lattice.PLAN_FLIPS)


def test_fuzz_gate_passes_a_few_random_specifications_on_the_host_learner():
    import numpy as np

    import fuzz  # noqa: E402

    rng = np.random.default_rng(5)
    specs = [fuzz.sample_spec(rng) for _ in range(4)]
    for s in specs:
        s["rows"] = min(s["rows"], 4000); s["rounds"] = min(s["rounds"], 10); s["cols"] = min(s["cols"], 40)
        fails, _ = fuzz.check_spec(s, "cpu")
        assert not fails, (fails, s)


def test_every_openmp_region_names_its_team_size():
    """A parallel region without ``num_threads`` takes the runtime's default team; a region with a smaller team than
    the previous one makes libgomp end the surplus workers and start them again for the next larger one (measured:
    240 us per region against 2.5 us). Every region therefore names its team: the full one or a single thread.
    Reference: .ci/check-omp-pragmas.sh (the same lint)."""
    import re
    from pathlib import Path

    root = Path(__file__).resolve().parents[1] / "falcata_b200" / "csrc"
    bad = []
    for path in list(root.rglob("*.cpp")) + list(root.rglob("*.cu")) + list(root.rglob("*.h")) + list(root.rglob("*.cuh")):
        if "build" in path.relative_to(root).parts:
            continue
        for no, line in enumerate(path.read_text().splitlines(), 1):
            if re.search(r"#\s*pragma\s+omp\s+parallel", line) and "num_threads(" not in line:
                bad.append(f"{path.relative_to(root)}:{no}")
    assert not bad, bad


def test_parameter_reference_is_up_to_date():
    """docs/Parameters.md is generated from the native parameter table; a parameter added to config.h without running the
    generator fails here."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, str(root / "docs" / "gen_parameters.py"), "--check"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
