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
