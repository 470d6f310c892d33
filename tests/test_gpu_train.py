"""Device training end to end: parity with the host learner, quality, predict kernel, device ingest."""
import numpy as np
import pytest
import torch

import falcata_b200 as fb
from util import auc, make_binary, make_multiclass, make_ranking, make_regression, model_body

pytestmark = pytest.mark.gpu


def _l2_exact(preds, data):
    lab = data.get_label()
    if hasattr(preds, "is_cuda"):
        lab = torch.as_tensor(lab, device=preds.device)
        return preds - lab, torch.ones_like(preds)
    return preds - lab, np.ones_like(preds)


@pytest.mark.parametrize("quant", ["stochastic", "fixedpoint"])
def test_first_tree_bit_identical_to_host(quant):
    # with custom L2 gradients and a zero start score both arms see exactly the same float gradients:
    # integer histograms + shared split math must then give the same tree, digit for digit
    X, y = make_regression(20000, 12)
    y = np.round(y * 8) / 8
    base = {"objective": "none", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": quant, "grow_policy": "level", "min_data_in_leaf": 20, "seed": 3}
    bc = fb.train({**base, "device_type": "cpu"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    bg = fb.train({**base, "device_type": "cuda"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    assert model_body(bc.model_to_string()) == model_body(bg.model_to_string())


@pytest.mark.parametrize("quant", ["none", "stochastic"])
def test_binary_quality_matches_host(quant):
    X, y = make_binary(30000, 28)
    p = {"objective": "binary", "num_leaves": 63, "max_bin": 63, "verbosity": -1, "quant_mode": quant, "grow_policy": "level"}
    bc = fb.train({**p, "device_type": "cpu"}, fb.Dataset(X[:25000], y[:25000]), 40)
    bg = fb.train({**p, "device_type": "cuda"}, fb.Dataset(X[:25000], y[:25000]), 40)
    ac, ag = auc(y[25000:], bc.predict(X[25000:])), auc(y[25000:], bg.predict(X[25000:]))
    assert ag > 0.93 and abs(ac - ag) < 0.01, (ac, ag)


def test_quant_run_twice_identical_and_device_ingest():
    X, y = make_binary(20000, 20)
    p = {"objective": "binary", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "device_type": "cuda"}
    a = fb.train(p, fb.Dataset(X, y), 15).model_to_string()
    b = fb.train(p, fb.Dataset(X, y), 15).model_to_string()
    assert a == b
    # device-array ingest bins on the GPU; same bins as host ingest -> same model
    c = fb.train(p, fb.Dataset(torch.from_numpy(X).cuda(), y, params={"bin_construct_sample_cnt": 20000}), 15).model_to_string()
    d = fb.train(p, fb.Dataset(X, y, params={"bin_construct_sample_cnt": 20000}), 15).model_to_string()
    assert model_body(c) == model_body(d)


@pytest.mark.parametrize("flip", ["device_controller:off", "fused_tail:off", "fused_scan:off", "fused_tail:off,fused_scan:off", "hist_lane:off", "col_major_part:off", "gh_in_row:on", "bulk_root:off", "hist_tc:on", "hist_lane_red:off"])
def test_plan_flips_keep_quantized_model_identical(flip):
    # performance-only plan keys must not change a single digit of a quantized model
    X, y = make_binary(30000, 20)
    p = {"objective": "binary", "num_leaves": 63, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "device_type": "cuda", "min_data_in_leaf": 5}
    a = fb.train(dict(p, cuda_plan="auto"), fb.Dataset(X, y), 8).model_to_string()
    b = fb.train(dict(p, cuda_plan="auto," + flip), fb.Dataset(X, y), 8).model_to_string()
    assert model_body(a) == model_body(b)


def test_device_predict_matches_host():
    X, y = make_binary(20000, 16)
    bst = fb.train({"objective": "binary", "num_leaves": 31, "verbosity": -1, "device_type": "cuda", "quant_mode": "stochastic"}, fb.Dataset(X, y), 30)
    ph = bst.predict(X)
    pd = bst.predict(torch.from_numpy(X).cuda())
    assert pd.is_cuda
    np.testing.assert_allclose(pd.cpu().numpy(), ph, atol=2e-5)
    raw = bst.predict(torch.from_numpy(X).cuda(), raw_score=True).cpu().numpy()
    np.testing.assert_allclose(raw, bst.predict(X, raw_score=True), atol=1e-4)


def test_validation_metrics_on_device():
    X, y = make_binary(20000, 16)
    ds = fb.Dataset(X[:16000], y[:16000]); dv = ds.create_valid(X[16000:], y[16000:])
    res = {}
    bst = fb.train({"objective": "binary", "metric": "binary_logloss,auc", "verbosity": -1, "device_type": "cuda", "quant_mode": "stochastic"}, ds, 25, valid_sets=[dv],
                   callbacks=[fb.record_evaluation(res)])
    ll = res["valid_0"]["binary_logloss"]
    assert ll[-1] < ll[0]
    p = bst.predict(X[16000:])
    ref = -np.mean(np.where(y[16000:] > 0, np.log(p), np.log(1 - p)))
    assert abs(ref - ll[-1]) < 1e-4
    assert abs(res["valid_0"]["auc"][-1] - auc(y[16000:], p)) < 1e-6


def test_regression_multiclass_ranking_on_device():
    X, y = make_regression(20000, 10)
    bst = fb.train({"objective": "regression", "verbosity": -1, "device_type": "cuda", "quant_mode": "fixedpoint"}, fb.Dataset(X[:16000], y[:16000]), 60)
    assert np.mean((bst.predict(X[16000:]) - y[16000:]) ** 2) < 0.3 * np.var(y)
    X, y = make_multiclass(20000, 12, 4)
    bst = fb.train({"objective": "multiclass", "num_class": 4, "verbosity": -1, "device_type": "cuda"}, fb.Dataset(X[:16000], y[:16000]), 30)
    p = bst.predict(X[16000:])
    assert p.shape == (4000, 4) and (p.argmax(1) == y[16000:]).mean() > 0.6
    X, y, g = make_ranking(500, 20, 10)
    res = {}
    fb.train({"objective": "lambdarank", "metric": "ndcg", "eval_at": "5", "verbosity": -1, "device_type": "cuda", "min_data_in_leaf": 5}, fb.Dataset(X, y, group=g), 30,
             valid_sets=[fb.Dataset(X, y, group=g)], callbacks=[fb.record_evaluation(res)])
    nd = res["valid_0"]["ndcg@5"]
    assert nd[-1] > nd[0] and nd[-1] > 0.8


@pytest.mark.parametrize("extra", [{"bagging_fraction": 0.6}, {"pos_bagging_fraction": 0.5, "neg_bagging_fraction": 0.9}])
def test_device_bagging_draws_the_host_bag(extra):
    # same Philox draw on both sides: with exact L2 gradients the first bagged tree is the same digit for digit
    X, y = make_regression(20000, 12)
    y = np.round(y * 8) / 8
    base = {"objective": "none", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "grow_policy": "level", "min_data_in_leaf": 20,
            "seed": 3, "bagging_freq": 1, **extra}
    bc = fb.train({**base, "device_type": "cpu"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    bg = fb.train({**base, "device_type": "cuda"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    assert model_body(bc.model_to_string()) == model_body(bg.model_to_string())


def test_device_bagging_trains_and_scores_out_of_bag_rows():
    X, y = make_binary(30000, 20)
    p = {"objective": "binary", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "device_type": "cuda", "bagging_fraction": 0.5,
         "bagging_freq": 2, "metric": "binary_logloss"}
    res = {}
    ds = fb.Dataset(X[:25000], y[:25000])
    bst = fb.train(p, ds, 30, valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(res)])
    # the training metric is computed from the device scores of ALL rows: it must agree with a fresh prediction
    pr = bst.predict(X[:25000])
    ref = -np.mean(np.where(y[:25000] > 0, np.log(pr), np.log(1 - pr)))
    assert abs(ref - res["train"]["binary_logloss"][-1]) < 1e-4
    assert auc(y[25000:], bst.predict(X[25000:])) > 0.9


def _make_categorical(n, seed=11):
    rng = np.random.RandomState(seed)
    Xn = rng.randn(n, 6).astype(np.float32)
    c_small = rng.randint(0, 3, size=n)          # 3 categories -> one-vs-rest
    c_big = rng.randint(0, 40, size=n)           # 40 categories -> sorted many-vs-many
    eff = rng.randn(40)
    y = (Xn[:, 0] + 0.5 * Xn[:, 1] * Xn[:, 2] + eff[c_big] + (c_small == 1) * 0.8 + 0.3 * rng.randn(n)).astype(np.float32)
    X = np.column_stack([Xn, c_small.astype(np.float32), c_big.astype(np.float32)])
    return X, y


@pytest.mark.parametrize("quant", ["stochastic", "none"])
def test_categorical_search_on_device_matches_host(quant):
    X, y = _make_categorical(20000)
    y = np.round(y * 8) / 8
    base = {"objective": "none", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": quant, "grow_policy": "level", "min_data_in_leaf": 20, "seed": 3,
            "min_data_per_group": 50, "cat_smooth": 10.0}
    mk = lambda: fb.Dataset(X, y, categorical_feature=[6, 7], free_raw_data=False)
    bc = fb.train({**base, "device_type": "cpu"}, mk(), 1, fobj=_l2_exact)
    bg = fb.train({**base, "device_type": "cuda"}, mk(), 1, fobj=_l2_exact)
    sc, sg = bc.model_to_string(), bg.model_to_string()
    assert "cat_threshold" in sg       # the device tree really uses categorical splits
    if quant == "stochastic":
        assert model_body(sc) == model_body(sg)
    else:
        np.testing.assert_allclose(bg.predict(X), bc.predict(X), atol=1e-4)


def test_categorical_training_and_device_predict():
    X, y = _make_categorical(30000)
    p = {"objective": "regression", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "device_type": "cuda", "metric": "l2"}
    ds = fb.Dataset(X[:25000], y[:25000], categorical_feature=[6, 7])
    dv = ds.create_valid(X[25000:], y[25000:])
    res = {}
    bst = fb.train(p, ds, 40, valid_sets=[dv], callbacks=[fb.record_evaluation(res)])
    ph = bst.predict(X[25000:])
    # validation scores are kept by binned traversal on the device: they must agree with the host walk on raw values
    assert abs(np.mean((ph - y[25000:]) ** 2) - res["valid_0"]["l2"][-1]) < 1e-3
    assert np.mean((ph - y[25000:]) ** 2) < 0.4 * np.var(y)
    pd = bst.predict(torch.from_numpy(X[25000:]).cuda()).cpu().numpy()
    np.testing.assert_allclose(pd, ph, atol=2e-4)


def test_compact_column_view_keeps_the_model():
    # feature_fraction 0.3: each tree constructs from a dense copy of its sampled columns only; same model as
    # constructing from the full rows
    X, y = make_binary(30000, 40)
    p = {"objective": "binary", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "device_type": "cuda", "feature_fraction": 0.3,
         "min_data_in_leaf": 5}
    a = fb.train(dict(p, cuda_plan="auto"), fb.Dataset(X, y), 8).model_to_string()
    b = fb.train(dict(p, cuda_plan="auto,compact_view:off"), fb.Dataset(X, y), 8).model_to_string()
    assert model_body(a) == model_body(b)
    assert len({int(t) for line in a.splitlines() if line.startswith("split_feature=") for t in line.split("=")[1].split()}) > 12


def test_leaf_renewal_on_device():
    # (a) quantized training with leaf values renewed from the true gradients: close to the host arm and to the
    #     un-renewed quantized model (stochastic rounding is unbiased, so neither is systematically better)
    X, y = make_regression(20000, 10)
    p = {"objective": "regression", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "quant_bins": 4, "grow_policy": "level"}
    mse = lambda b: float(np.mean((b.predict(X) - y) ** 2))
    plain = fb.train({**p, "device_type": "cuda"}, fb.Dataset(X, y), 20)
    renew = fb.train({**p, "device_type": "cuda", "quant_train_renew_leaf": True}, fb.Dataset(X, y), 20)
    host = fb.train({**p, "device_type": "cpu", "quant_train_renew_leaf": True}, fb.Dataset(X, y), 20)
    assert renew.model_to_string() != plain.model_to_string() and mse(renew) < 1.1 * mse(plain)
    assert abs(mse(renew) - mse(host)) < 0.05 * mse(host)
    # (b) L1 regression: leaf values are medians of the residuals (objective-side renewal)
    yl = y + (np.random.RandomState(3).rand(len(y)) < 0.05) * 50.0   # heavy outliers
    pl = {"objective": "regression_l1", "num_leaves": 31, "verbosity": -1, "grow_policy": "level"}
    dev = fb.train({**pl, "device_type": "cuda"}, fb.Dataset(X, yl), 30)
    cpu = fb.train({**pl, "device_type": "cpu"}, fb.Dataset(X, yl), 30)
    mae = lambda b: float(np.mean(np.abs(b.predict(X) - yl)))
    assert abs(mae(dev) - mae(cpu)) < 0.05 * mae(cpu)


def test_goss_on_device():
    X, y = make_binary(30000, 20)
    p = {"objective": "binary", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "data_sample_strategy": "goss", "top_rate": 0.2,
         "other_rate": 0.1, "learning_rate": 0.2, "metric": "binary_logloss"}
    res = {}
    ds = fb.Dataset(X[:25000], y[:25000])
    dev = fb.train({**p, "device_type": "cuda"}, ds, 40, valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(res)])
    cpu = fb.train({**p, "device_type": "cpu"}, fb.Dataset(X[:25000], y[:25000]), 40)
    ad, ac = auc(y[25000:], dev.predict(X[25000:])), auc(y[25000:], cpu.predict(X[25000:]))
    assert ad > 0.93 and abs(ad - ac) < 0.01, (ad, ac)
    # the sampled trees really are smaller samples: leaf counts of a late tree add up to about (top + other) of the rows
    late = dev.dump_model()["tree_info"][-1]["tree_structure"]
    total = late["internal_count"]
    assert 0.25 * 25000 < total < 0.36 * 25000, total
    # scores of out-of-sample rows are kept up to date (training metric equals a fresh prediction)
    pr = dev.predict(X[:25000])
    ref = -np.mean(np.where(y[:25000] > 0, np.log(pr), np.log(1 - pr)))
    assert abs(ref - res["train"]["binary_logloss"][-1]) < 1e-4


def test_device_ndcg_matches_a_plain_computation():
    X, y, g = make_ranking(300, 25, 10)
    res = {}
    ds = fb.Dataset(X, y, group=g)
    bst = fb.train({"objective": "lambdarank", "metric": "ndcg", "eval_at": "3,10", "verbosity": -1, "device_type": "cuda", "min_data_in_leaf": 5}, ds, 10,
                   valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(res)])
    s = bst.predict(X, raw_score=True)
    out = {3: [], 10: []}
    pos = 0
    for cnt in g:
        sc, lab = s[pos:pos + cnt], y[pos:pos + cnt]; pos += cnt
        order = np.argsort(-sc, kind="stable"); ideal = np.argsort(-lab, kind="stable")
        for k in (3, 10):
            disc = 1.0 / np.log2(2.0 + np.arange(min(k, cnt)))
            dcg = np.sum((2.0 ** lab[order[:k]] - 1) * disc); idcg = np.sum((2.0 ** lab[ideal[:k]] - 1) * disc)
            out[k].append(dcg / idcg if idcg > 0 else 1.0)
    assert abs(np.mean(out[3]) - res["train"]["ndcg@3"][-1]) < 1e-5
    assert abs(np.mean(out[10]) - res["train"]["ndcg@10"][-1]) < 1e-5


def test_extra_trees_on_device_matches_host():
    # one random threshold per (tree, leaf, feature), drawn from a counter-based generator: both arms evaluate the
    # same thresholds, so the first tree is the same digit for digit
    X, y = make_regression(20000, 12)
    y = np.round(y * 8) / 8
    base = {"objective": "none", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "grow_policy": "level", "min_data_in_leaf": 20,
            "seed": 3, "extra_trees": True}
    bc = fb.train({**base, "device_type": "cpu"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    bg = fb.train({**base, "device_type": "cuda"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    plain = fb.train({**base, "device_type": "cuda", "extra_trees": False}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    assert model_body(bc.model_to_string()) == model_body(bg.model_to_string())
    assert model_body(bg.model_to_string()) != model_body(plain.model_to_string())


@pytest.mark.parametrize("ff", [1.0, 0.4])
def test_four_bit_packed_view_keeps_the_model(ff):
    # max_bin 15: every group fits a nibble, the construct kernel reads a two-groups-per-byte copy of the sampled columns
    X, y = make_binary(30000, 37)
    p = {"objective": "binary", "num_leaves": 31, "max_bin": 15, "verbosity": -1, "quant_mode": "stochastic", "device_type": "cuda", "feature_fraction": ff,
         "min_data_in_leaf": 5}
    mk = lambda: fb.Dataset(X, y, params={"max_bin": 15})
    a = fb.train(dict(p, cuda_plan="auto"), mk(), 8).model_to_string()
    b = fb.train(dict(p, cuda_plan="auto,pack4:off,compact_view:off"), mk(), 8).model_to_string()
    assert model_body(a) == model_body(b)


@pytest.mark.parametrize("objective", ["mape", "cross_entropy_lambda", "multi_regression"])
def test_gradient_kernels_of_mape_xentlambda_and_multi_regression_match_the_host_objective(objective, monkeypatch):
    """These three objectives have device gradient kernels; FALCATA_HOST_GRADIENTS=1 sends the same training through
    the objective's host code (scores down, gradients up). Both routes must give the same trees."""
    rng = np.random.default_rng(5)
    n = 12000
    X = rng.normal(size=(n, 8)).astype(np.float32)
    extra = {}
    if objective == "mape":
        y = (np.abs(X[:, 0] * 3 + X[:, 1]) + 0.5).astype(np.float32)
    elif objective == "cross_entropy_lambda":
        y = (1.0 / (1.0 + np.exp(-(X[:, 0] + 0.5 * X[:, 1])))).astype(np.float32)
    else:
        y = np.column_stack([X[:, 0] + 0.1 * rng.normal(size=n), -2 * X[:, 1] + X[:, 2]]).astype(np.float32)
        extra = {"num_class": 2}
    w = rng.uniform(0.5, 2.0, size=n).astype(np.float32)
    p = {"objective": objective, "num_leaves": 15, "verbosity": -1, "device_type": "cuda", "quant_mode": "none", "min_data_in_leaf": 20, **extra}
    kernel = fb.train(p, fb.Dataset(X, y, weight=w), 6)
    monkeypatch.setenv("FALCATA_HOST_GRADIENTS", "1")
    host = fb.train(p, fb.Dataset(X, y, weight=w), 6)
    monkeypatch.delenv("FALCATA_HOST_GRADIENTS")
    a, b = np.asarray(kernel.predict(X, raw_score=True)), np.asarray(host.predict(X, raw_score=True))
    assert np.max(np.abs(a - b)) < 1e-4 * (1.0 + np.max(np.abs(b)))
    sk = [t["tree_structure"].get("split_feature") for t in kernel.dump_model()["tree_info"]]
    sh = [t["tree_structure"].get("split_feature") for t in host.dump_model()["tree_info"]]
    assert sk == sh


def test_mape_on_the_device_reaches_the_host_learners_loss():
    X, y = make_regression(15000, 8)
    y = np.abs(y) + 1.0
    p = {"objective": "mape", "num_leaves": 15, "verbosity": -1, "grow_policy": "level", "metric": "mape"}
    dev = fb.train({**p, "device_type": "cuda"}, fb.Dataset(X, y), 30)
    cpu = fb.train({**p, "device_type": "cpu"}, fb.Dataset(X, y), 30)
    mape = lambda b: float(np.mean(np.abs(b.predict(X) - y) / np.maximum(1.0, np.abs(y))))
    assert abs(mape(dev) - mape(cpu)) < 0.05 * mape(cpu) + 1e-3


def test_host_matrix_is_binned_on_the_device_with_the_host_bins():
    # a numpy matrix that trains on the device goes through chunk copies and the binning kernel; the bin sample is
    # the same Philox draw as on the host path, so both ingests give the same bins and the same model
    X, y = make_binary(260000, 10)       # more rows than the bin sample (200k): the draw matters
    p = {"objective": "binary", "num_leaves": 15, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "device_type": "cuda"}
    dev_ingest = fb.Dataset(X, y)
    a = fb.train(p, dev_ingest, 5)
    assert dev_ingest.info()["has_host"] == 0 and dev_ingest.info()["has_device"] == 1
    host_ingest = fb.Dataset(X, y, params={"keep_host_bins": True})
    b = fb.train(p, host_ingest, 5)
    assert host_ingest.info()["has_host"] == 1
    assert model_body(a.model_to_string()) == model_body(b.model_to_string())
    t = fb.train(p, fb.Dataset(torch.from_numpy(X).pin_memory(), y), 5)
    assert model_body(t.model_to_string()) == model_body(a.model_to_string())


def test_bundled_sparse_features_match_host():
    # mutually exclusive sparse columns are bundled into shared byte columns (EFB); the device binner, construct,
    # search (most-frequent-bin reconstruction) and partition must treat the bundles exactly like the host learner
    rng = np.random.RandomState(5)
    n = 20000
    dense = rng.randn(n, 4).astype(np.float32)
    which = rng.randint(0, 12, size=n)
    sparse = np.zeros((n, 12), dtype=np.float32)
    sparse[np.arange(n), which] = rng.randint(1, 6, size=n)          # one non-zero per row: 12 exclusive features
    X = np.column_stack([dense, sparse])
    y = np.round((dense[:, 0] + 0.7 * (which % 3) + 0.2 * sparse.sum(1) + 0.1 * rng.randn(n)) * 8) / 8
    base = {"objective": "none", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "grow_policy": "level", "min_data_in_leaf": 20, "seed": 3}
    dc = fb.Dataset(X, y, free_raw_data=False); dg = fb.Dataset(X, y, free_raw_data=False)
    bc = fb.train({**base, "device_type": "cpu"}, dc, 2, fobj=_l2_exact)
    bg = fb.train({**base, "device_type": "cuda"}, dg, 2, fobj=_l2_exact)
    assert dg.info()["num_groups"] < 16 and dg.info()["num_groups"] == dc.info()["num_groups"]     # bundling happened, the same on both paths
    sc, sg = bc.model_to_string(), bg.model_to_string()
    assert model_body(sc).split("Tree=1")[0] == model_body(sg).split("Tree=1")[0]
    used = {int(t) for line in sg.splitlines() if line.startswith("split_feature=") for t in line.split("=")[1].split()}
    assert any(f >= 4 for f in used)      # bundled features are split on


def test_monotone_constraints_on_device():
    # every split orders its children and the device controller hands the output ranges down the subtree,
    # so the prediction is monotone in a constrained feature whatever the other features are
    rng = np.random.default_rng(3)
    n = 20000
    X = rng.normal(size=(n, 4)).astype(np.float32)
    y = (np.sin(2 * X[:, 0]) + 0.5 * X[:, 0] - np.cos(2 * X[:, 1]) - 0.3 * X[:, 1] + X[:, 2] * X[:, 0] * 0.5
         + 0.1 * rng.normal(size=n)).astype(np.float32)
    p = {"objective": "regression", "num_leaves": 31, "learning_rate": 0.2, "verbosity": -1, "min_data_in_leaf": 10,
         "monotone_constraints": [1, -1, 0, 0], "device_type": "cuda"}
    b = fb.train(p, fb.Dataset(torch.as_tensor(X, device="cuda"), y), 30)

    def worst(bst, col, sign):
        base = rng.normal(size=(200, 4)).astype(np.float32)
        prev, w = None, 0.0
        for g in np.linspace(-3, 3, 41, dtype=np.float32):
            A = base.copy()
            A[:, col] = g
            pr = bst.predict(A).astype(np.float64)
            if prev is not None:
                w = max(w, float(np.max(sign * (prev - pr))))
            prev = pr
        return w

    assert worst(b, 0, +1) <= 1e-10 and worst(b, 1, -1) <= 1e-10
    free = fb.train({**p, "monotone_constraints": [0, 0, 0, 0]}, fb.Dataset(torch.as_tensor(X, device="cuda"), y), 30)
    assert worst(free, 0, +1) > 1e-3
    mse_c = float(np.mean((b.predict(X) - y) ** 2))
    assert mse_c < 0.6 * float(np.var(y))   # the constrained model still learns


@pytest.mark.parametrize("case", ["bynode", "interaction", "both"])
def test_per_node_feature_masks_on_device_match_host(case):
    # the device draws the host learner's per-node sample (same Philox keys, same k) and applies the same
    # interaction sets, so with identical gradients the first tree is the host's tree
    X, y = make_regression(20000, 12)
    y = np.round(y * 8) / 8
    base = {"objective": "none", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "grow_policy": "level", "min_data_in_leaf": 20, "seed": 3}
    if case in ("bynode", "both"):
        base["feature_fraction_bynode"] = 0.5
    if case in ("interaction", "both"):
        base["interaction_constraints"] = "[0,1,2,3],[3,4,5,6,7],[8,9,10]"
    else:
        base["quant_mode"] = "stochastic"
    bc = fb.train({**base, "device_type": "cpu"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    bg = fb.train({**base, "device_type": "cuda"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    assert bc.num_trees() == 1 and "num_leaves=31" in bc.model_to_string()
    if "quant_mode" in base:
        assert model_body(bc.model_to_string()) == model_body(bg.model_to_string())
    else:
        # float histograms: sums differ in the last digits between host and device, the structure must not
        def structure(m):
            return [ln for ln in m.model_to_string().splitlines() if ln.startswith(("split_feature=", "threshold=", "left_child=", "right_child="))]
        assert structure(bc) == structure(bg)


@pytest.mark.parametrize("leaves", [15, 63])
def test_leafwise_growth_on_device_is_the_host_best_first_tree(leaves):
    # grow_policy=leaf: the device over-grows level by level (a leaf is split while it ranks among the best
    # num_leaves-1 nodes by the smallest gain on its path) and the host keeps the best-first tree; with identical
    # gradients and integer histograms that is the host leaf-wise learner's tree, digit for digit
    X, y = make_regression(30000, 12)
    y = np.round(y * 8) / 8
    base = {"objective": "none", "num_leaves": leaves, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "grow_policy": "leaf",
            "min_data_in_leaf": 20, "seed": 3}
    bc = fb.train({**base, "device_type": "cpu"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    bg = fb.train({**base, "device_type": "cuda"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    assert f"num_leaves={leaves}" in bc.model_to_string()
    assert model_body(bc.model_to_string()) == model_body(bg.model_to_string())
    lvl = fb.train({**base, "device_type": "cuda", "grow_policy": "level"}, fb.Dataset(X, y, free_raw_data=False), 1, fobj=_l2_exact)
    assert model_body(lvl.model_to_string()) != model_body(bg.model_to_string())


@pytest.mark.parametrize("extra", [{}, {"bagging_fraction": 0.6, "bagging_freq": 1}, {"quant_train_renew_leaf": True}, {"objective": "regression_l1"}])
def test_leafwise_growth_trains_and_scores_consistently(extra):
    # several rounds: the score update runs through the final tree's leaf windows, so the training metric the
    # device reports must equal the metric of predict() on the same rows
    X, y = make_binary(40000, 16)
    p = {"objective": "binary", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": "stochastic", "grow_policy": "leaf",
         "device_type": "cuda", "metric": "binary_logloss", "min_data_in_leaf": 20, **extra}
    if p["objective"] == "regression_l1":
        # leaf outputs renewed by the objective (medians through the final tree's leaf windows)
        p["metric"] = "l1"
        ds = fb.Dataset(X, y, free_raw_data=False)
        ev = {}
        b = fb.train(p, ds, 20, valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(ev)])
        assert abs(float(np.mean(np.abs(b.predict(X) - y))) - ev["train"]["l1"][-1]) < 1e-5
        assert ev["train"]["l1"][-1] < 0.8 * ev["train"]["l1"][0]
        return
    ds = fb.Dataset(X, y, free_raw_data=False)
    ev = {}
    b = fb.train(p, ds, 20, valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(ev)])
    pr = np.clip(b.predict(X), 1e-15, 1 - 1e-15)
    ll = float(-np.mean(y * np.log(pr) + (1 - y) * np.log(1 - pr)))
    assert abs(ll - ev["train"]["binary_logloss"][-1]) < 1e-5
    assert auc(y, pr) > 0.9


def test_linear_tree_with_cuda_inputs_falls_back_to_the_host():
    # linear leaves are fitted and evaluated on the host; CUDA tensors and device_type=cuda are accepted all the same
    rng = np.random.default_rng(0)
    X = rng.normal(size=(6000, 5)).astype(np.float32)
    y = np.where(X[:, 0] > 0, 2 * X[:, 1] + 1, -3 * X[:, 2]).astype(np.float32)
    p = {"objective": "regression", "num_leaves": 8, "learning_rate": 0.2, "linear_tree": True, "verbosity": -1, "device_type": "cuda"}
    Xd = torch.as_tensor(X, device="cuda")
    b = fb.train(p, fb.Dataset(Xd, y, params=p), 20)
    pd = b.predict(Xd)
    assert pd.is_cuda and "is_linear=1" in b.model_to_string()
    ph = b.predict(X)
    assert np.allclose(pd.cpu().numpy(), ph, atol=1e-5)
    assert float(np.mean((ph - y) ** 2)) < 0.05
    reloaded = fb.Booster(model_str=b.model_to_string())
    assert np.allclose(reloaded.predict(Xd).cpu().numpy(), ph, atol=1e-5)


def test_multi_regression_on_the_device_engine():
    """Several regression targets on the device: trees are grown by the device engine (gradients come from the host
    objective), and every target's column equals a single-target device model."""
    rng = np.random.default_rng(23)
    n = 5000
    X = rng.normal(size=(n, 8)).astype(np.float32)
    Y = np.column_stack([X[:, 0] + 0.1 * rng.normal(size=n), -2 * X[:, 1] + X[:, 2] + 5.0])
    p = {"objective": "multi_regression", "num_class": 2, "num_leaves": 15, "verbosity": -1, "device_type": "cuda", "quant_mode": "none", "metric": "l2"}
    rec = {}
    ds = fb.Dataset(X, Y)
    bst = fb.train(p, ds, 10, valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(rec)])
    pred = np.asarray(bst.predict(X))
    assert pred.shape == (n, 2) and bst.num_trees() == 20
    assert rec["train"]["l2"][-1] < 0.3 * rec["train"]["l2"][0]
    assert abs(rec["train"]["l2"][-1] - np.mean((pred - Y.astype(np.float32)) ** 2)) < 1e-4
    for t in range(2):
        one = fb.train({"objective": "regression", "num_leaves": 15, "verbosity": -1, "device_type": "cuda", "quant_mode": "none"}, fb.Dataset(X, Y[:, t]), 10)
        np.testing.assert_allclose(pred[:, t], one.predict(X), rtol=1e-4, atol=1e-4)


def test_more_than_255_bins_with_a_device_booster_fall_back_to_the_host_learner():
    rng = np.random.default_rng(31)
    X = rng.normal(size=(6000, 4)).astype(np.float32); y = np.sin(3 * X[:, 0]) + 0.05 * rng.normal(size=6000)
    p = {"objective": "regression", "num_leaves": 63, "max_bin": 1023, "verbosity": -1, "min_data_in_leaf": 5, "min_data_in_bin": 1}
    dev = fb.train(dict(p, device_type="cuda"), fb.Dataset(X, y, params={"max_bin": 1023, "min_data_in_bin": 1}), 10)
    host = fb.train(dict(p, device_type="cpu"), fb.Dataset(X, y, params={"max_bin": 1023, "min_data_in_bin": 1}), 10)
    assert model_body(dev.model_to_string()) == model_body(host.model_to_string())


@pytest.mark.parametrize("objective,extra", [("regression_l1", {}), ("quantile", {"alpha": 0.8})])
def test_percentile_leaf_renewal_on_the_device_matches_the_host_path(objective, extra):
    """L1 / quantile leaves are renewed from a per-leaf percentile of the residuals: the segmented-sort kernel path
    gives the values of the host computation on downloaded scores."""
    import os
    rng = np.random.default_rng(41)
    X = rng.normal(size=(20000, 8)).astype(np.float32)
    y = X[:, 0] * 2 + np.abs(X[:, 1]) + rng.standard_t(3, size=20000)
    p = dict({"objective": objective, "num_leaves": 31, "verbosity": -1, "device_type": "cuda", "quant_mode": "none", "learning_rate": 0.2}, **extra)
    dev = fb.train(p, fb.Dataset(X, y), 12)
    os.environ["FALCATA_RENEW_ON_HOST"] = "1"
    try:
        host = fb.train(p, fb.Dataset(X, y), 12)
    finally:
        del os.environ["FALCATA_RENEW_ON_HOST"]
    np.testing.assert_allclose(dev.predict(X), host.predict(X), rtol=1e-9, atol=1e-9)
    med = np.median(y - dev.predict(X)) if objective == "regression_l1" else np.quantile(y - dev.predict(X), 0.8)
    assert abs(med) < 0.1


def test_rank_xendcg_gradient_kernel_matches_the_host_objective():
    """rank_xendcg on the device: the kernel makes the host objective's random draws (keyed on row, round, seed) and its
    three-pass gradient; training with it and with host-computed gradients gives the same ranking quality and nearly
    the same scores."""
    import os
    rng = np.random.default_rng(51)
    q, per = 300, 40
    n = q * per
    X = rng.normal(size=(n, 10)).astype(np.float32)
    s = X[:, 0] - 0.5 * X[:, 1] + 0.3 * rng.normal(size=n)
    y = np.zeros(n, dtype=np.float32)
    for i in range(q):
        seg = s[i * per:(i + 1) * per]
        y[i * per:(i + 1) * per] = np.digitize(seg, np.quantile(seg, [0.5, 0.75, 0.9, 0.97]))
    group = np.full(q, per, dtype=np.int32)
    p = {"objective": "rank_xendcg", "metric": "ndcg", "eval_at": [5], "num_leaves": 15, "verbosity": -1, "device_type": "cuda", "quant_mode": "none",
         "min_data_in_leaf": 10, "learning_rate": 0.1}

    def run():
        rec = {}
        ds = fb.Dataset(X, y, group=group)
        b = fb.train(p, ds, 15, valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(rec)])
        return b.predict(X), rec["train"]["ndcg@5"]
    pd, nd = run()
    os.environ["FALCATA_HOST_GRADIENTS"] = "1"
    try:
        ph, nh = run()
    finally:
        del os.environ["FALCATA_HOST_GRADIENTS"]
    assert nd[-1] > nd[0] and nd[-1] > 0.75
    assert abs(nd[-1] - nh[-1]) < 0.02
    assert np.corrcoef(pd, ph)[0, 1] > 0.99


def test_monotone_penalty_on_the_device_matches_the_host_learner():
    rng = np.random.default_rng(71)
    X = rng.normal(size=(8000, 3)).astype(np.float32); y = 3 * X[:, 0] + X[:, 1] + 0.1 * rng.normal(size=8000)
    p = {"objective": "regression", "num_leaves": 15, "verbosity": -1, "min_data_in_leaf": 10, "monotone_constraints": [1, 0, 0], "monotone_penalty": 2.0,
         "quant_mode": "none"}
    dev = fb.train(dict(p, device_type="cuda"), fb.Dataset(X, y), 3)
    host = fb.train(dict(p, device_type="cpu"), fb.Dataset(X, y), 3)
    root = lambda b: b.dump_model()["tree_info"][0]["tree_structure"]["split_feature"]
    assert root(dev) != 0 and root(dev) == root(host)
    np.testing.assert_allclose(dev.predict(X), host.predict(X), rtol=1e-5, atol=1e-5)


def test_plan_tuner_probes_the_device_and_keeps_the_model(tmp_path, monkeypatch):
    from falcata_b200 import tuner

    monkeypatch.setenv("FALCATA_WISDOM", str(tmp_path / "wisdom.json"))
    X, y = make_binary(60000, 12)
    params = {"objective": "binary", "num_leaves": 31, "verbosity": -1, "quant_mode": "stochastic", "quant_bins": 4, "device_type": "cuda"}
    plan = tuner.tune(params, fb.Dataset(X, y), rounds=4, warmup=2, switches=["fused_scan", "fused_tail", "hist_lane_red"])
    assert plan.startswith("auto")
    entry = tuner.load_wisdom()[tuner.wisdom_key(params, 60000, 12)]
    assert entry["plan"] == plan and len(entry["probes"]) == 4 and all("ms" in p for p in entry["probes"])
    a = fb.train(dict(params, cuda_plan="wisdom"), fb.Dataset(X, y), 6).model_to_string()
    b = fb.train(dict(params), fb.Dataset(X, y), 6).model_to_string()
    assert model_body(a) == model_body(b)


def test_self_verify_mode_checks_device_binning_and_tiled_predict():
    """FALCATA_VERIFY=1: device binning is compared with the host's bin mappers on sampled rows and the tiled predict
    kernel with the general one; FALCATA_DEBUG=diag prints the construct geometry and a line per tree (reference:
    tests/gates/README.md:L41-42, src/treelearner/cuda/plan.h:L286-322)."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    code = (
        "import torch, numpy as np, falcata_b200 as fb\n"
        "g = torch.Generator(device='cuda').manual_seed(1)\n"
        "X = torch.randn(50000, 12, device='cuda', generator=g); X[::7, 3] = float('nan'); X[:, 5] = torch.randint(0, 9, (50000,), device='cuda', generator=g).float()\n"
        "y = ((X[:, 0] + X[:, 1] * X[:, 2]) > 0).float().cpu().numpy()\n"
        "p = {'objective': 'binary', 'num_leaves': 31, 'max_bin': 63, 'verbosity': 1, 'device_type': 'cuda', 'categorical_feature': [5]}\n"
        "b = fb.train(p, fb.Dataset(X, y, categorical_feature=[5]), 3)\n"
        "q = {'objective': 'binary', 'num_leaves': 31, 'max_bin': 63, 'verbosity': 1, 'device_type': 'cuda'}\n"
        "b2 = fb.train(q, fb.Dataset(X[:, :5].contiguous(), y), 3)\n"
        "pr = b2.predict(X[:, :5].contiguous())\n"
        "print('DONE', float(pr.mean()))\n")
    env = dict(os.environ, FALCATA_VERIFY="1", FALCATA_DEBUG="diag", PYTHONPATH=str(Path(__file__).resolve().parents[1]))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    text = out.stdout + out.stderr
    assert out.returncode == 0, text[-3000:]
    assert "DONE" in text
    assert text.count("FALCATA_VERIFY: device binning equals the host's on 1024 sampled rows") >= 2
    assert "FALCATA_VERIFY: tiled predict equals the general kernel on 50000 scores" in text
    assert "[diag] construct: lane mode" in text and "[diag] tree 0:" in text


def test_c_api_dataset_from_a_device_matrix_matches_the_python_route():
    """FB_DatasetCreateFromDeviceMat (the reference's FLC_DatasetCreateFromMatDevice): sample gathered on the device, bin
    boundaries on the host, rows binned on the device. Trains to the model of `fb.Dataset(cuda_tensor)`, which draws the
    same sample by row id; a column-major matrix and a reference dataset give the same bins."""
    import ctypes

    from falcata_b200.basic import _lib, _safe_call

    lib = _lib()
    X, y = make_binary(30000, 10)
    Xd = torch.as_tensor(X, device="cuda").contiguous()
    params = "max_bin=63 verbosity=-1"
    train = "objective=binary num_leaves=31 max_bin=63 verbosity=-1 device_type=cuda quant_mode=stochastic seed=5"

    def train_on(handle, rounds=5):
        yy = np.ascontiguousarray(y, dtype=np.float32)
        _safe_call(lib.FB_DatasetSetField(handle, b"label", yy.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(len(yy)), 0))
        bst = ctypes.c_void_p()
        _safe_call(lib.FB_BoosterCreate(handle, train.encode(), ctypes.byref(bst)))
        fin = ctypes.c_int()
        for _ in range(rounds):
            _safe_call(lib.FB_BoosterUpdateOneIter(bst, ctypes.byref(fin)))
        n = ctypes.c_int64()
        _safe_call(lib.FB_BoosterSaveModelToString(bst, 0, -1, 0, ctypes.c_int64(0), ctypes.byref(n), None))
        buf = ctypes.create_string_buffer(n.value)
        _safe_call(lib.FB_BoosterSaveModelToString(bst, 0, -1, 0, ctypes.c_int64(n.value), ctypes.byref(n), buf))
        _safe_call(lib.FB_BoosterFree(bst))
        return buf.value.decode()

    h1 = ctypes.c_void_p()
    _safe_call(lib.FB_DatasetCreateFromDeviceMat(ctypes.c_void_p(Xd.data_ptr()), 0, ctypes.c_int32(Xd.shape[0]), ctypes.c_int32(Xd.shape[1]), 1, params.encode(), None, ctypes.byref(h1)))
    m1 = train_on(h1)
    # column-major copy of the same matrix, bins taken from the first dataset
    Xc = Xd.t().contiguous()
    h2 = ctypes.c_void_p()
    _safe_call(lib.FB_DatasetCreateFromDeviceMat(ctypes.c_void_p(Xc.data_ptr()), 0, ctypes.c_int32(Xd.shape[0]), ctypes.c_int32(Xd.shape[1]), 0, params.encode(), h1, ctypes.byref(h2)))
    m2 = train_on(h2)
    assert model_body(m1) == model_body(m2)
    py = fb.train({"objective": "binary", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "device_type": "cuda", "quant_mode": "stochastic", "seed": 5},
                  fb.Dataset(Xd, y, params={"max_bin": 63}), 5)
    assert model_body(py.model_to_string()) == model_body(m1)
    _safe_call(lib.FB_DatasetFree(h2)); _safe_call(lib.FB_DatasetFree(h1))


@pytest.mark.parametrize("quant", ["fixedpoint", "none"])
def test_forced_splits_on_the_device_match_the_host_learner(tmp_path, quant):
    """forcedsplits_filename on one GPU: the tree grows under the host's control and the forced nodes' records are
    evaluated on the host from the leaf's histogram in the device pool. With integer histograms the model is the host
    learner's, digit for digit (same forced top, same leaf numbering); with real-valued bins the trees agree in
    structure. A forced node on a feature with missing values and one that cannot be applied are part of the file."""
    import json

    X, y = make_regression(20000, 8)
    X = X.copy(); X[::9, 2] = np.nan
    y = np.round(y * 8) / 8
    forced = {"feature": 3, "threshold": 0.25,
              "left": {"feature": 2, "threshold": -0.5, "left": {"feature": 5, "threshold": 0.1}},
              "right": {"feature": 1, "threshold": 0.0, "right": {"feature": 6, "threshold": 1e9}}}   # the last one leaves nothing on the right: ignored
    path = tmp_path / "forced.json"
    path.write_text(json.dumps(forced))
    base = {"objective": "none", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "quant_mode": quant, "grow_policy": "level", "min_data_in_leaf": 20, "seed": 3,
            "forcedsplits_filename": str(path)}
    if quant != "none":
        base["quant_bins"] = 64
    bc = fb.train({**base, "device_type": "cpu"}, fb.Dataset(X, y, free_raw_data=False), 2, fobj=_l2_exact)
    bg = fb.train({**base, "device_type": "cuda"}, fb.Dataset(X, y, free_raw_data=False), 2, fobj=_l2_exact)
    for t in bg.dump_model()["tree_info"]:
        root = t["tree_structure"]
        assert root["split_feature"] == 3 and root["left_child"]["split_feature"] == 2 and root["right_child"]["split_feature"] == 1
        assert root["left_child"]["left_child"]["split_feature"] == 5
        assert t["num_leaves"] == 31
    if quant != "none":
        assert model_body(bc.model_to_string()) == model_body(bg.model_to_string())
    else:
        sc, sg = bc.dump_model()["tree_info"][0]["tree_structure"], bg.dump_model()["tree_info"][0]["tree_structure"]
        assert sc["split_feature"] == sg["split_feature"] and sc["threshold"] == sg["threshold"]
        assert np.max(np.abs(bc.predict(X) - bg.predict(X))) < 1e-3


def test_dart_on_the_device_engine_follows_the_host_learner():
    """boosting=dart with device_type=cuda: trees grow on the device; dropped trees leave and re-enter the device's
    training scores by binned traversal (validation scores are rescaled in place). Same drop draws as the host
    learner, so with integer histograms the two models agree tree for tree; the recorded validation metric is the
    metric of the final model's predictions."""
    Xa, ya = make_binary(25000, 10)
    X, y, Xv, yv = Xa[:20000], ya[:20000], Xa[20000:], ya[20000:]
    p = {"objective": "binary", "boosting": "dart", "drop_rate": 0.3, "skip_drop": 0.2, "num_leaves": 15, "max_bin": 63, "verbosity": -1, "quant_mode": "fixedpoint",
         "quant_bins": 64, "min_data_in_leaf": 20, "metric": "binary_logloss", "seed": 7}
    rec = {}
    dtrain = fb.Dataset(X, y, free_raw_data=False)
    dev = fb.train({**p, "device_type": "cuda"}, dtrain, 25, valid_sets=[fb.Dataset(Xv, yv, reference=dtrain)], valid_names=["v"], callbacks=[fb.record_evaluation(rec)])
    cpu = fb.train({**p, "device_type": "cpu"}, fb.Dataset(X, y, free_raw_data=False), 25)
    assert dev.num_trees() == 25
    pd_, pc = np.asarray(dev.predict(Xv)), np.asarray(cpu.predict(Xv))
    assert np.max(np.abs(pd_ - pc)) < 2e-3
    ll = float(-np.mean(yv * np.log(np.clip(pd_, 1e-15, 1)) + (1 - yv) * np.log(np.clip(1 - pd_, 1e-15, 1))))
    assert abs(rec["v"]["binary_logloss"][-1] - ll) < 2e-4     # the device's validation scores followed every rescaling
    assert auc(yv, pd_) > 0.75


def test_random_forest_on_the_device_engine_follows_the_host_learner():
    """boosting=rf with device_type=cuda: every tree is trained on the device on the gradients at the start score; the
    device scores hold the running mean of the trees (each carrying the start score). Same bags as the host learner:
    with integer histograms both forests predict alike, and the recorded metric is the final forest's."""
    Xa, ya = make_binary(25000, 10)
    X, y, Xv, yv = Xa[:20000], ya[:20000], Xa[20000:], ya[20000:]
    p = {"objective": "binary", "boosting": "rf", "bagging_freq": 1, "bagging_fraction": 0.6, "feature_fraction": 0.8, "num_leaves": 31, "max_bin": 63, "verbosity": -1,
         "quant_mode": "fixedpoint", "quant_bins": 64, "min_data_in_leaf": 20, "metric": "binary_logloss", "seed": 3}
    rec = {}
    dtrain = fb.Dataset(X, y, free_raw_data=False)
    dev = fb.train({**p, "device_type": "cuda"}, dtrain, 12, valid_sets=[fb.Dataset(Xv, yv, reference=dtrain)], valid_names=["v"], callbacks=[fb.record_evaluation(rec)])
    cpu = fb.train({**p, "device_type": "cpu"}, fb.Dataset(X, y, free_raw_data=False), 12)
    assert dev.num_trees() == 12
    pd_, pc = np.asarray(dev.predict(Xv)), np.asarray(cpu.predict(Xv))
    assert np.max(np.abs(pd_ - pc)) < 2e-3
    ll = float(-np.mean(yv * np.log(np.clip(pd_, 1e-15, 1)) + (1 - yv) * np.log(np.clip(1 - pd_, 1e-15, 1))))
    assert abs(rec["v"]["binary_logloss"][-1] - ll) < 2e-4
    assert auc(yv, pd_) > 0.8


def test_linear_trees_on_a_device_booster_follow_the_host_learner():
    """linear_tree with device_type=cuda (one GPU, no row sampling): the trees grow on the device, the leaf regressions
    are solved on the host from the raw values and the device scores take the difference by row. With integer
    histograms the trees are the host learner's, so the predictions agree closely; the recorded validation loss is the
    loss of the final model's predictions (the device scores followed every linear correction)."""
    rng = np.random.default_rng(0)
    n = 8000

    def target(A):
        return np.where(A[:, 0] > 0, 2 * A[:, 1] + 1, -3 * A[:, 2]).astype(np.float32)

    X = rng.normal(size=(n, 5)).astype(np.float32)
    y = target(X) + 0.05 * rng.normal(size=n).astype(np.float32)
    Xv = rng.normal(size=(2000, 5)).astype(np.float32)
    Xv[::50, 1] = np.nan
    yv = target(np.nan_to_num(Xv))
    out = {}
    for dev in ("cpu", "cuda"):
        p = {"objective": "regression", "num_leaves": 8, "learning_rate": 0.2, "linear_tree": True, "linear_lambda": 0.01, "verbose": -1, "min_data_in_leaf": 20,
             "device_type": dev, "quant_mode": "fixedpoint", "quant_bins": 64, "max_bin": 63}
        ds = fb.Dataset(X, y, params=p)
        dv = fb.Dataset(Xv, yv, reference=ds)
        ev = {}
        b = fb.train(p, ds, 20, valid_sets=[dv], valid_names=["v"], callbacks=[fb.record_evaluation(ev)])
        pr = b.predict(Xv)
        out[dev] = (pr, ev["v"]["l2"][-1], b)
        assert "is_linear=1" in b.model_to_string()
    assert abs(out["cuda"][1] - float(np.mean((out["cuda"][0] - yv) ** 2))) < 1e-4
    assert np.max(np.abs(out["cuda"][0] - out["cpu"][0])) < 5e-3
    constant = fb.train({"objective": "regression", "num_leaves": 8, "learning_rate": 0.2, "verbose": -1, "min_data_in_leaf": 20, "device_type": "cuda", "max_bin": 63},
                        fb.Dataset(X, y), 20)
    assert float(np.mean((out["cuda"][0] - yv) ** 2)) < 0.5 * float(np.mean((constant.predict(Xv) - yv) ** 2))
