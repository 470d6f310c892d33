"""The command-line application against the Python API on the same files.
Parity: tests/python_package_test/test_consistency.py (CLI vs Python on the example configs)."""
import os
import subprocess

import numpy as np

import falcata_b200 as fb
from falcata_b200.libpath import find_lib_path


def _exe():
    return os.path.join(os.path.dirname(os.path.dirname(find_lib_path())), "bin", "falcata")


def _run(cwd, *args):
    r = subprocess.run([_exe(), *args], cwd=cwd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout + r.stderr


def test_cli_train_predict_convert_refit(tmp_path):
    rng = np.random.RandomState(0)
    X = rng.randn(3000, 6); y = (X[:, 0] + X[:, 1] * X[:, 2] > 0).astype(int)
    np.savetxt(tmp_path / "train.csv", np.column_stack([y[:2400], X[:2400]]), delimiter=",", fmt="%.17g")
    np.savetxt(tmp_path / "valid.csv", np.column_stack([y[2400:], X[2400:]]), delimiter=",", fmt="%.17g")
    (tmp_path / "train.conf").write_text("task = train\nobjective = binary\ndata = train.csv\nvalid = valid.csv\nnum_trees = 20\nnum_leaves = 15\n"
                                         "metric = auc\nmetric_freq = 5\nsnapshot_freq = 10\noutput_model = model.txt\ndevice_type = cpu  # host learner\nverbosity = 1\n")
    out = _run(tmp_path, "config=train.conf")
    assert "Iteration:20, valid_1 auc" in out and (tmp_path / "model.txt.snapshot_iter_10").exists()
    # command-line arguments override the file
    _run(tmp_path, "config=train.conf", "num_trees=3", "output_model=small.txt")
    assert fb.Booster(model_file=str(tmp_path / "small.txt")).num_trees() == 3
    # same parameters through the Python API give the same model
    ds = fb.Dataset(str(tmp_path / "train.csv"), params={"header": False})
    py = fb.train({"objective": "binary", "num_leaves": 15, "device_type": "cpu", "verbosity": -1}, ds, 20)
    cli = fb.Booster(model_file=str(tmp_path / "model.txt"))
    np.testing.assert_allclose(cli.predict(X[2400:]), py.predict(X[2400:]), rtol=1e-9)
    _run(tmp_path, "task=predict", "input_model=model.txt", "data=valid.csv", "output_result=pred.txt")
    np.testing.assert_allclose(np.loadtxt(tmp_path / "pred.txt"), cli.predict(X[2400:]), rtol=1e-6)
    _run(tmp_path, "task=convert_model", "input_model=model.txt", "convert_model_language=cpp", "convert_model=m.cpp")
    assert "double" in (tmp_path / "m.cpp").read_text()
    _run(tmp_path, "task=refit", "input_model=model.txt", "data=valid.csv", "output_model=refit.txt", "objective=binary")
    assert fb.Booster(model_file=str(tmp_path / "refit.txt")).num_trees() == 20
    _run(tmp_path, "task=save_binary", "data=train.csv")
    assert (tmp_path / "train.csv.bin").exists()


def test_native_core_unit_tests_pass():
    """The C++ unit tests of the core library (formatting, binning, tree round trip, split math, best-first order keys)."""
    import subprocess
    from pathlib import Path
    import falcata_b200
    from falcata_b200 import build as fbuild
    fbuild.build()
    exe = Path(falcata_b200.__file__).parent / "bin" / "falcata_core_tests"
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert " 0 failed" in r.stdout


def _free_ports(k):
    import socket

    socks = [socket.socket() for _ in range(k)]
    for s in socks:
        s.bind(("127.0.0.1", 0))
    ports = [s.getsockname()[1] for s in socks]
    for s in socks:
        s.close()
    return ports


def test_cli_distributed_training_over_tcp(tmp_path):
    """The command line's distributed mode (reference: tests/distributed/_test_distributed.py): one process per machine list
    entry on 127.0.0.1, collectives over TCP, pre-partitioned data files, tree_learner=data. With integer histograms the
    processes write the model that a single process trains on the whole file, digit for digit; a shared file that every
    process splits by itself (pre_partition=false) gives the same model again; three processes with the voting learner
    agree with one another."""
    from util import model_body

    rng = np.random.RandomState(3)
    n = 6000
    X = rng.randn(n, 8); y = (X[:, 0] + X[:, 1] * X[:, 2] + 0.3 * rng.randn(n) > 0).astype(int)
    full = np.column_stack([y, X])
    np.savetxt(tmp_path / "train.txt", full, delimiter="\t", fmt="%.17g")
    common = ("task = train\nobjective = binary\nnum_trees = 8\nnum_leaves = 15\nmin_data_in_leaf = 20\nmax_bin = 63\nquant_mode = fixedpoint\nquant_bins = 64\n"
              "verbosity = 1\nnum_threads = 2\n")
    (tmp_path / "single.conf").write_text(common + "data = train.txt\noutput_model = single.txt\ndevice_type = cpu\n")
    _run(tmp_path, "config=single.conf")
    single = (tmp_path / "single.txt").read_text()

    def launch(world, extra, files, tag):
        ports = _free_ports(world)
        (tmp_path / f"mlist_{tag}.txt").write_text("".join(f"127.0.0.1 {p}\n" for p in ports))
        procs = []
        for r in range(world):
            (tmp_path / f"{tag}{r}.conf").write_text(common + extra + f"data = {files[r]}\noutput_model = {tag}{r}.txt\nlocal_listen_port = {ports[r]}\n"
                                                     f"num_machines = {world}\nmachine_list_file = mlist_{tag}.txt\ntime_out = 1\n")
            procs.append(subprocess.Popen([_exe(), f"config={tag}{r}.conf"], cwd=tmp_path, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        outs = []
        for p in procs:
            try:
                o, _ = p.communicate(timeout=240)
            except subprocess.TimeoutExpired:
                for q in procs:
                    q.kill()
                raise
            outs.append(o)
            assert p.returncode == 0, o
        return [(tmp_path / f"{tag}{r}.txt").read_text() for r in range(world)], outs

    # two pre-partitioned files
    np.savetxt(tmp_path / "part0.txt", full[: n // 2], delimiter="\t", fmt="%.17g")
    np.savetxt(tmp_path / "part1.txt", full[n // 2:], delimiter="\t", fmt="%.17g")
    models, outs = launch(2, "pre_partition = true\ntree_learner = data\n", ["part0.txt", "part1.txt"], "pp")
    assert "this is rank" in outs[0]
    assert model_body(models[0]) == model_body(models[1]) == model_body(single)
    # one shared file, every process keeps its block of rows
    models, _ = launch(2, "pre_partition = false\ntree_learner = data\n", ["train.txt", "train.txt"], "sh")
    assert model_body(models[0]) == model_body(models[1]) == model_body(single)
    # feature-parallel: every process loads the whole file and searches its share of the features
    models, _ = launch(2, "tree_learner = feature\n", ["train.txt", "train.txt"], "fp")
    assert model_body(models[0]) == model_body(models[1]) == model_body(single)
    # three processes, voting
    thirds = np.array_split(full, 3)
    for r in range(3):
        np.savetxt(tmp_path / f"third{r}.txt", thirds[r], delimiter="\t", fmt="%.17g")
    models, _ = launch(3, "pre_partition = true\ntree_learner = voting\ntop_k = 4\n", [f"third{r}.txt" for r in range(3)], "vt")
    assert model_body(models[0]) == model_body(models[1]) == model_body(models[2])
    pr = fb.Booster(model_str=models[0]).predict(X)
    assert float(np.mean((pr > 0.5) == y)) > 0.85


def test_examples_run(tmp_path):
    """The Python quick start (host learner here) and the command-line example files keep working."""
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "quickstart.py"), "--device", "cpu", "--rows", "6000", "--rounds", "10"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "same predictions" in r.stdout, r.stdout + r.stderr
    rng = np.random.RandomState(1)
    X = rng.randn(2000, 10); y = (X[:, 0] + X[:, 1] * X[:, 2] > 0).astype(int)
    os.makedirs(tmp_path / "examples" / "cli")
    np.savetxt(tmp_path / "examples" / "cli" / "train.tsv", np.column_stack([y[:1600], X[:1600]]), delimiter="\t", fmt="%.9g")
    np.savetxt(tmp_path / "examples" / "cli" / "valid.tsv", np.column_stack([y[1600:], X[1600:]]), delimiter="\t", fmt="%.9g")
    for name in ("train.conf", "predict.conf"):
        out = _run(tmp_path, "config=" + os.path.join(root, "examples", "cli", name), "num_trees=10")
    assert "Finished prediction" in out and len(np.loadtxt(tmp_path / "examples" / "cli" / "predictions.txt")) == 400
    # the torchrun example with two CPU workers: both ranks report the model that one process trains
    import re

    multi = os.path.join(root, "examples", "multi_gpu.py")
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nproc-per-node", "2", multi, "--device", "cpu",
                          "--rows", "12000", "--rounds", "4"], capture_output=True, text=True, timeout=600)
    one = subprocess.run([sys.executable, multi, "--device", "cpu", "--rows", "12000", "--rounds", "4"], capture_output=True, text=True, timeout=600)
    md5s = re.findall(r"model md5 ([0-9a-f]{32})", two.stdout + two.stderr) + re.findall(r"model md5 ([0-9a-f]{32})", one.stdout + one.stderr)
    assert len(md5s) == 3 and len(set(md5s)) == 1, two.stdout + two.stderr + one.stdout + one.stderr
