"""Device prediction: the tiled kernel (rows staged in shared memory, trees streamed through it in chunks) and the
general node-array kernel against the host traversal: raw scores, converted scores, leaf indices."""
import os

import numpy as np
import pytest
import torch

import falcata_b200 as fb

pytestmark = pytest.mark.gpu


def _data(n, f, seed=0, nan_frac=0.0, zero_frac=0.0):
    rng = np.random.default_rng(seed)
    X = rng.normal(size=(n, f)).astype(np.float32)
    if zero_frac:
        X[rng.random(size=X.shape) < zero_frac] = 0.0
    if nan_frac:
        X[rng.random(size=X.shape) < nan_frac] = np.nan
    return X, rng


@pytest.mark.parametrize("n,f,leaves,rounds", [(1, 5, 7, 3), (255, 5, 7, 3), (257, 40, 31, 20), (30011, 136, 255, 40)])
@pytest.mark.parametrize("missing", ["none", "nan", "zero"])
def test_tiled_predict_matches_host(n, f, leaves, rounds, missing):
    X, rng = _data(max(n, 4000), f, nan_frac=0.1 if missing == "nan" else 0.0, zero_frac=0.3 if missing == "zero" else 0.0)
    y = (np.nan_to_num(X[:, 0]) + 0.5 * np.nan_to_num(X[:, 1]) * np.nan_to_num(X[:, 2]) + 0.1 * rng.normal(size=X.shape[0]) > 0).astype(np.float32)
    p = {"objective": "binary", "num_leaves": leaves, "verbosity": -1, "min_data_in_leaf": 5, "zero_as_missing": missing == "zero", "use_missing": missing != "none"}
    bst = fb.train(p, fb.Dataset(X, y), rounds)
    Xp = X[:n]
    Xd = torch.from_numpy(Xp).cuda()
    raw_h = bst.predict(Xp, raw_score=True)
    raw_d = bst.predict(Xd, raw_score=True)
    assert raw_d.is_cuda
    np.testing.assert_allclose(raw_d.cpu().numpy().reshape(-1), np.asarray(raw_h).reshape(-1), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(bst.predict(Xd).cpu().numpy().reshape(-1), np.asarray(bst.predict(Xp)).reshape(-1), atol=2e-5)
    leaf_h = bst.predict(Xp, pred_leaf=True)
    leaf_d = bst.predict(Xd, pred_leaf=True)
    assert leaf_d.is_cuda and leaf_d.dtype == torch.int32
    assert np.array_equal(leaf_d.cpu().numpy(), np.asarray(leaf_h).reshape(n, -1))
    # a range of iterations
    if rounds >= 6:
        a = bst.predict(Xd, raw_score=True, start_iteration=2, num_iteration=3).cpu().numpy()
        np.testing.assert_allclose(a.reshape(-1), np.asarray(bst.predict(Xp, raw_score=True, start_iteration=2, num_iteration=3)).reshape(-1), rtol=1e-5, atol=1e-5)
        assert np.array_equal(bst.predict(Xd, pred_leaf=True, start_iteration=2, num_iteration=3).cpu().numpy(),
                              np.asarray(bst.predict(Xp, pred_leaf=True, start_iteration=2, num_iteration=3)).reshape(n, -1))
    # the general kernel gives the same scores
    os.environ["FALCATA_PREDICT_GENERAL"] = "1"
    try:
        raw_g = bst.predict(Xd, raw_score=True)
    finally:
        del os.environ["FALCATA_PREDICT_GENERAL"]
    np.testing.assert_allclose(raw_g.cpu().numpy(), raw_d.cpu().numpy(), rtol=1e-5, atol=1e-5)


def test_tiled_predict_multiclass_and_dtypes():
    X, rng = _data(6000, 20, seed=4)
    y = np.argmax(X[:, :4] + 0.3 * rng.normal(size=(6000, 4)), axis=1).astype(np.float32)
    bst = fb.train({"objective": "multiclass", "num_class": 4, "num_leaves": 15, "verbosity": -1}, fb.Dataset(X, y), 12)
    ph = np.asarray(bst.predict(X))
    for t in (torch.from_numpy(X).cuda(), torch.from_numpy(X.astype(np.float64)).cuda()):
        pd = bst.predict(t)
        assert tuple(pd.shape) == (6000, 4)
        np.testing.assert_allclose(pd.cpu().numpy(), ph, atol=3e-5)
    leaf_d = bst.predict(torch.from_numpy(X).cuda(), pred_leaf=True).cpu().numpy()
    assert np.array_equal(leaf_d, np.asarray(bst.predict(X, pred_leaf=True)).reshape(6000, -1))


def test_predict_with_categorical_forest_takes_general_kernel():
    rng = np.random.default_rng(5)
    X = rng.normal(size=(5000, 6)).astype(np.float32)
    X[:, 3] = rng.integers(0, 12, size=5000)
    y = ((X[:, 3] % 3 == 0) ^ (X[:, 0] > 0)).astype(np.float32)
    bst = fb.train({"objective": "binary", "num_leaves": 15, "verbosity": -1, "min_data_per_group": 10, "cat_smooth": 1.0}, fb.Dataset(X, y, categorical_feature=[3]), 10)
    assert "decision_type=1" in bst.model_to_string() or "cat_boundaries" in bst.model_to_string()
    Xd = torch.from_numpy(X).cuda()
    np.testing.assert_allclose(bst.predict(Xd, raw_score=True).cpu().numpy(), bst.predict(X, raw_score=True), rtol=1e-5, atol=1e-5)
    # leaf indices of a forest the device kernel does not cover come from the host, as a device tensor all the same
    leaf = bst.predict(Xd, pred_leaf=True)
    assert leaf.is_cuda and np.array_equal(leaf.cpu().numpy(), np.asarray(bst.predict(X, pred_leaf=True)).reshape(5000, -1))


def test_nan_inputs_to_a_forest_without_missing_handling_read_as_zero():
    """A forest trained on complete data has no missing-aware node: NaN at prediction time is taken as 0, on the host
    and in the device kernel's comparison-only walk."""
    X, rng = _data(5000, 12, seed=9)
    y = (X[:, 0] - X[:, 1] > 0).astype(np.float32)
    bst = fb.train({"objective": "binary", "num_leaves": 31, "verbosity": -1}, fb.Dataset(X, y), 15)
    Xn = X.copy(); Xn[rng.random(size=Xn.shape) < 0.2] = np.nan
    host = bst.predict(Xn, raw_score=True)
    dev = bst.predict(torch.from_numpy(Xn).cuda(), raw_score=True).cpu().numpy()
    np.testing.assert_allclose(dev, host, rtol=1e-5, atol=1e-5)
    assert np.array_equal(bst.predict(torch.from_numpy(Xn).cuda(), pred_leaf=True).cpu().numpy(), np.asarray(bst.predict(Xn, pred_leaf=True)).reshape(5000, -1))
