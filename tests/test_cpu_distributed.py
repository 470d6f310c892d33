"""Multi-process CPU training over gloo: the host parallel learners against the single-process learner,
and failure detection when a rank dies on the host.
Parity: tests/distributed/_test_distributed.py:L53-190 (N processes on localhost compared with one)."""
import os
import socket
import subprocess
import sys

import pytest

import falcata_b200 as fb
from util import make_binary, model_body

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(world, extra, timeout=180):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dist_cpu_worker.py")] + extra, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
            o += "\nKILLED_BY_TEST_TIMEOUT"
        outs.append((p.returncode, o))
    return outs


def _single(learner_rows, quant, rounds):
    X, y = make_binary(learner_rows, 12)
    params = {"objective": "binary", "num_leaves": 15, "max_bin": 63, "verbosity": -1, "device_type": "cpu", "grow_policy": "level", "quant_mode": quant,
              "min_data_in_leaf": 5, "seed": 5}
    return fb.train(params, fb.Dataset(X, y).set_global_rows(0, learner_rows), rounds).model_to_string()


@pytest.mark.parametrize("learner,quant", [("data", "stochastic"), ("feature", "stochastic"), ("voting", "stochastic"), ("data", "none")])
def test_two_ranks_match_single_process(tmp_path, learner, quant):
    out = str(tmp_path / "model.txt")
    res = _launch(2, ["--learner", learner, "--quant", quant, "--out", out])
    for rc, o in res:
        assert rc == 0, o[-2000:]
    dist_model = open(out).read()
    single = _single(6000, quant, 10)
    if quant == "stochastic":
        # integer histograms: the sharded sum is exact, so the model is the same digit for digit
        assert model_body(dist_model) == model_body(single)
    else:
        a = fb.Booster(model_str=dist_model); b = fb.Booster(model_str=single)
        X, _ = make_binary(6000, 12)
        import numpy as np

        assert np.abs(a.predict(X) - b.predict(X)).max() < 1e-3


def test_rank_that_dies_is_detected_on_the_host():
    res = _launch(2, ["--mode", "fail"], timeout=90)
    assert res[1][0] == 7
    rc0, o0 = res[0]
    assert "KILLED_BY_TEST_TIMEOUT" not in o0, o0[-2000:]
    assert rc0 != 0 and ("TRAIN_ERROR" in o0 or "Error" in o0), o0[-2000:]


_TCP_WORKER = r"""
import sys, numpy as np
sys.path.insert(0, {root!r})
import falcata_b200 as fb
rank, ports = int(sys.argv[1]), [int(p) for p in sys.argv[2].split(",")]
rng = np.random.RandomState(5)
n = 6000
X = rng.randn(n, 8); y = (X[:, 0] + X[:, 1] * X[:, 2] + 0.3 * rng.randn(n) > 0).astype(np.float64)
lo, hi = (0, n) if rank < 0 else (n * rank // len(ports), n * (rank + 1) // len(ports))
p = {{"objective": "binary", "num_leaves": 15, "min_data_in_leaf": 20, "max_bin": 63, "quant_mode": "fixedpoint", "quant_bins": 64, "verbosity": -1,
     "device_type": "cpu", "num_threads": 2}}
if rank >= 0:
    p.update(tree_learner="data", num_machines=len(ports), machines=",".join(f"127.0.0.1:{{q}}" for q in ports), local_listen_port=ports[rank], time_out=1)
b = fb.train(p, fb.Dataset(X[lo:hi], y[lo:hi]), 6)
if rank >= 0:
    b.free_network()
print("MODEL_BEGIN"); print(b.model_to_string().split("\nparameters:")[0]); print("MODEL_END")
"""


def test_python_api_trains_over_the_tcp_mesh_like_one_process(tmp_path):
    """A machine list in the training parameters (num_machines, machines, local_listen_port) makes every process join the
    TCP mesh before its Dataset is binned: the processes exchange their pieces of the one global bin sample and number
    their rows in machine-list order. With integer histograms two processes holding half of the rows each train the model
    that one process trains on all rows, digit for digit."""
    import socket
    import subprocess
    import sys
    from pathlib import Path

    root = str(Path(__file__).resolve().parents[1])
    script = tmp_path / "worker.py"
    script.write_text(_TCP_WORKER.format(root=root))
    socks = [socket.socket() for _ in range(2)]
    for s in socks:
        s.bind(("127.0.0.1", 0))
    ports = ",".join(str(s.getsockname()[1]) for s in socks)
    for s in socks:
        s.close()

    def model_of(out):
        return out.split("MODEL_BEGIN\n")[1].split("MODEL_END")[0]

    single = subprocess.run([sys.executable, str(script), "-1", ports], capture_output=True, text=True, timeout=300)
    assert single.returncode == 0, single.stdout + single.stderr
    procs = [subprocess.Popen([sys.executable, str(script), str(r), ports], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for pr in procs:
        try:
            o, _ = pr.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        assert pr.returncode == 0, o
        outs.append(o)
    assert model_of(outs[0]) == model_of(outs[1]) == model_of(single.stdout)


def test_a_process_that_leaves_the_tcp_mesh_ends_the_others_with_an_error(tmp_path):
    """Failure detection on the TCP mesh, made on the host: one process exits right after the mesh is up; the other's next
    collective finds the connection closed and comes back with an error instead of waiting."""
    import socket
    import subprocess
    import sys
    from pathlib import Path

    root = str(Path(__file__).resolve().parents[1])
    script = tmp_path / "leaver.py"
    script.write_text(
        "import os, sys, numpy as np\n"
        f"sys.path.insert(0, {root!r})\n"
        "import falcata_b200 as fb\n"
        "rank, ports = int(sys.argv[1]), [int(p) for p in sys.argv[2].split(',')]\n"
        "fb.network_init(','.join(f'127.0.0.1:{q}' for q in ports), ports[rank], 1, 2)\n"
        "if rank == 1:\n"
        "    os._exit(0)                      # leaves without a word\n"
        "rng = np.random.RandomState(0); X = rng.randn(2000, 5); y = (X[:, 0] > 0).astype(float)\n"
        "try:\n"
        "    fb.train({'objective': 'binary', 'tree_learner': 'data', 'device_type': 'cpu', 'verbosity': -1}, fb.Dataset(X, y), 3)\n"
        "except fb.FalcataError as e:\n"
        "    print('ERROR', e); sys.exit(5)\n"
        "print('trained'); sys.exit(0)\n")
    socks = [socket.socket() for _ in range(2)]
    for s in socks:
        s.bind(("127.0.0.1", 0))
    ports = ",".join(str(s.getsockname()[1]) for s in socks)
    for s in socks:
        s.close()
    procs = [subprocess.Popen([sys.executable, str(script), str(r), ports], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for pr in procs:
        try:
            o, _ = pr.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append((pr.returncode, o))
    assert outs[1][0] == 0
    assert outs[0][0] == 5 and "ERROR" in outs[0][1] and ("closed its connection" in outs[0][1] or "Socket" in outs[0][1]), outs[0][1]
