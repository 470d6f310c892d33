"""Multi-GPU data-parallel training: the quantized model must be bit-identical at any GPU count."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run_raw(world, out, extra=()):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", "29519",
           os.path.join(HERE, "multi_gpu_worker.py"), "--out", out, *extra]
    return subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=300)


def _run(world, out, extra=()):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if world == 1:
        cmd = [sys.executable, os.path.join(HERE, "multi_gpu_worker.py"), "--out", out, *extra]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", "29517",
               os.path.join(HERE, "multi_gpu_worker.py"), "--out", out, *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return open(out).read()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("quant", ["stochastic", "fixedpoint"])
def test_bit_identical_across_gpu_counts(tmp_path, quant):
    extra = ("--quant", quant)
    ref = _run(1, str(tmp_path / "m1.txt"), extra)
    assert "Tree=4" in ref
    worlds = [w for w in (2, 4, 8) if w <= torch.cuda.device_count()]
    for w in worlds:
        got = _run(w, str(tmp_path / f"m{w}.txt"), extra)
        assert got == ref, f"model differs at {w} GPUs"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_bit_identical_across_gpu_counts_at_benchmark_scale(tmp_path):
    # the shape of the headline benchmark per rank (millions of rows, 255 leaves, 8 levels deep, 20 rounds): small
    # data sets do not exercise full-width levels, multi-wave grids or cross-rank timing
    extra = ("--rows", "2200000", "--leaves", "255", "--rounds", "20")
    ref = _run(1, str(tmp_path / "m1.txt"), extra)
    assert "Tree=19" in ref
    for w in [w for w in (2, 4, 8) if w <= torch.cuda.device_count()]:
        assert _run(w, str(tmp_path / f"m{w}.txt"), extra) == ref, f"model differs at {w} GPUs"
    # the unfused level chain (separate argmax / gather / controller / scan launches) grows the same trees
    w = min(2, torch.cuda.device_count())
    assert _run(w, str(tmp_path / "m_unfused.txt"), extra + ("--plan", "auto,fused_tail:off,fused_scan:off")) == ref


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_leafwise_growth_bit_identical_across_gpu_counts(tmp_path):
    # exact leaf-wise growth: every rank's controller sees the same gathered best splits, over-grows the same
    # nodes and the host replay keeps the same tree, so the model is the single-GPU model at any GPU count
    extra = ("--grow-policy", "leaf", "--leaves", "63")
    ref = _run(1, str(tmp_path / "m1.txt"), extra)
    assert "Tree=4" in ref
    for w in [w for w in (2, 4, 8) if w <= torch.cuda.device_count()]:
        assert _run(w, str(tmp_path / f"m{w}.txt"), extra) == ref, f"model differs at {w} GPUs"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_leafwise_growth_feature_parallel_matches_single_gpu(tmp_path):
    extra = ("--grow-policy", "leaf", "--leaves", "63")
    ref = _run(1, str(tmp_path / "m1.txt"), extra)
    got = _run(2, str(tmp_path / "m2.txt"), ("--learner", "feature", *extra))
    assert got == ref


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("extra", [(), ("--categorical",)])
def test_feature_parallel_matches_single_gpu(tmp_path, extra):
    # rows replicated, features split between the ranks, split bitmaps broadcast by the owner of the split
    # feature: the model must be the single-GPU model, digit for digit
    ref = _run(1, str(tmp_path / "m1.txt"), extra)
    got = _run(2, str(tmp_path / "m2.txt"), ("--learner", "feature", *extra))
    assert got == ref


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_departed_rank_is_noticed_before_the_next_launch(tmp_path):
    r = _run_raw(2, str(tmp_path / "m.txt"), ("--skip-rank", "1", "--rounds", "50"))
    out = r.stdout + r.stderr
    assert "rank 1 leaves after round 2" in out
    assert "TRAIN_ERROR" in out and "left the job" in out, out[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_voting_with_every_feature_voted_matches_single_gpu(tmp_path):
    # top_k >= number of features: the vote keeps everything, so the restricted reduce-scatter carries all
    # features and the model must be the single-GPU model
    ref = _run(1, str(tmp_path / "m1.txt"))
    got = _run(2, str(tmp_path / "m2.txt"), ("--learner", "voting", "--top-k", "28"))
    assert got == ref


def _run_gloo(world, extra):
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT="29523", OMP_NUM_THREADS="4")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dist_cpu_worker.py"), *extra], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    for p in procs:
        o, _ = p.communicate(timeout=300)
        assert p.returncode == 0, o[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_voting_with_small_top_k_matches_the_host_voting_learner(tmp_path):
    # a real vote (3 of 12 features per rank): the device path must pick the features, reduce the bins and split
    # exactly like the host voting learner run on the same two shards. One tree: from the second tree on the
    # two arms see gradients that differ in the last float bit (host double vs device float sigmoid).
    from util import model_body

    common = ["--learner", "voting", "--quant", "stochastic", "--top-k", "3", "--rows", "40000", "--rounds", "1", "--leaves", "63"]
    _run_gloo(2, [*common, "--device", "cpu", "--out", str(tmp_path / "host.txt")])
    _run_gloo(2, [*common, "--device", "cuda", "--out", str(tmp_path / "dev.txt")])
    assert model_body(open(tmp_path / "dev.txt").read()) == model_body(open(tmp_path / "host.txt").read())
