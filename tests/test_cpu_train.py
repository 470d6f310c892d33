"""CPU end-to-end: training quality, model text / binary round trips, callbacks, cv."""
import numpy as np
import pytest

import falcata_b200 as fb
from util import auc, make_binary, make_multiclass, make_ranking, make_regression


def test_binary_config1_quality():
    X, y = make_binary()
    ds = fb.Dataset(X[:8000], y[:8000])
    bst = fb.train({"objective": "binary", "num_leaves": 31, "max_bin": 255, "learning_rate": 0.1, "device_type": "cpu", "verbosity": -1, "grow_policy": "leaf"}, ds, 100)
    p = bst.predict(X[8000:])
    assert auc(y[8000:], p) > 0.96


@pytest.mark.parametrize("policy", ["leaf", "level"])
@pytest.mark.parametrize("quant", ["none", "stochastic", "fixedpoint"])
def test_policies_and_quant(policy, quant):
    X, y = make_binary(6000, 12)
    ds = fb.Dataset(X[:5000], y[:5000])
    bst = fb.train({"objective": "binary", "num_leaves": 15, "device_type": "cpu", "verbosity": -1, "grow_policy": policy, "quant_mode": quant}, ds, 30)
    assert auc(y[5000:], bst.predict(X[5000:])) > 0.93
    # quantized training is deterministic
    bst2 = fb.train({"objective": "binary", "num_leaves": 15, "device_type": "cpu", "verbosity": -1, "grow_policy": policy, "quant_mode": quant}, fb.Dataset(X[:5000], y[:5000]), 30)
    assert bst.model_to_string() == bst2.model_to_string()


def test_model_roundtrips(tmp_path):
    X, y = make_binary(4000, 10)
    bst = fb.train({"objective": "binary", "device_type": "cpu", "verbosity": -1}, fb.Dataset(X, y), 20)
    s = bst.model_to_string()
    b2 = fb.Booster(model_str=s)
    assert b2.model_to_string() == s
    np.testing.assert_array_equal(bst.predict(X), b2.predict(X))
    f = tmp_path / "m.txt"
    bst.save_model(f)
    b3 = fb.Booster(model_file=f)
    np.testing.assert_array_equal(bst.predict(X), b3.predict(X))
    blob = bst.model_to_binary()
    assert blob[:4] == b"FALB" and len(blob) < len(s)
    b4 = fb.Booster.from_binary(blob)
    np.testing.assert_allclose(bst.predict(X), b4.predict(X), rtol=0, atol=1e-12)
    b5 = fb.Booster.from_binary(bst.model_to_binary(f32_leaves=True))
    np.testing.assert_allclose(bst.predict(X), b5.predict(X), atol=1e-5)
    d = bst.dump_model()
    assert len(d["tree_info"]) == 20 and d["max_feature_idx"] == 9
    assert "PredictTree0" in bst.model_to_if_else()


def test_model_text_format_fields():
    X, y = make_binary(2000, 6)
    s = fb.train({"objective": "binary", "device_type": "cpu", "verbosity": -1, "num_leaves": 7}, fb.Dataset(X, y), 3).model_to_string()
    lines = s.split("\n")
    assert lines[0] == "tree" and lines[1] == "version=v4"
    for key in ["num_class=1", "num_tree_per_iteration=1", "label_index=0", "max_feature_idx=5", "objective=binary sigmoid:1", "feature_names=", "feature_infos=", "tree_sizes=",
                "Tree=0", "num_leaves=", "num_cat=0", "split_feature=", "split_gain=", "threshold=", "decision_type=", "left_child=", "right_child=", "leaf_value=", "leaf_weight=",
                "leaf_count=", "internal_value=", "internal_weight=", "internal_count=", "is_linear=0", "shrinkage=", "end of trees", "feature_importances:", "parameters:", "end of parameters"]:
        assert any(l.startswith(key) for l in lines), key
    sizes = [int(v) for v in [l for l in lines if l.startswith("tree_sizes=")][0].split("=")[1].split()]
    body = s[s.index("Tree=0"):s.index("end of trees")]
    assert sum(sizes) == len(body)


def test_regression_multiclass_ranking():
    X, y = make_regression()
    bst = fb.train({"objective": "regression", "device_type": "cpu", "verbosity": -1}, fb.Dataset(X[:4000], y[:4000]), 80)
    assert np.mean((bst.predict(X[4000:]) - y[4000:]) ** 2) < 0.35 * np.var(y)
    X, y = make_multiclass()
    bst = fb.train({"objective": "multiclass", "num_class": 4, "device_type": "cpu", "verbosity": -1}, fb.Dataset(X[:5000], y[:5000]), 40)
    p = bst.predict(X[5000:])
    assert p.shape == (1000, 4) and np.allclose(p.sum(1), 1) and (p.argmax(1) == y[5000:]).mean() > 0.6
    X, y, g = make_ranking()
    res = {}
    fb.train({"objective": "lambdarank", "metric": "ndcg", "eval_at": "5", "device_type": "cpu", "verbosity": -1, "min_data_in_leaf": 5}, fb.Dataset(X, y, group=g), 30,
             valid_sets=[fb.Dataset(X, y, group=g)], callbacks=[fb.record_evaluation(res)])
    nd = res["valid_0"]["ndcg@5"]
    assert nd[-1] > nd[0] and nd[-1] > 0.8


def test_early_stopping_and_cv():
    X, y = make_binary(5000, 10)
    ds = fb.Dataset(X[:4000], y[:4000]); dv = ds.create_valid(X[4000:], y[4000:])
    bst = fb.train({"objective": "binary", "metric": "binary_logloss", "device_type": "cpu", "verbosity": -1, "learning_rate": 0.5, "num_leaves": 63, "min_data_in_leaf": 2}, ds, 300,
                   valid_sets=[dv], callbacks=[fb.early_stopping(5, verbose=False)])
    assert 0 < bst.best_iteration < 300
    r = fb.cv({"objective": "binary", "metric": "auc", "device_type": "cpu", "verbosity": -1}, fb.Dataset(X, y), 10, nfold=3)
    assert len(r["valid auc-mean"]) == 10 and r["valid auc-mean"][-1] > 0.9


def test_custom_objective_and_continue():
    X, y = make_regression(3000, 6)

    def l2(preds, data):
        return preds - data.get_label(), np.ones_like(preds)

    ds = fb.Dataset(X, y, free_raw_data=False)
    b1 = fb.train({"objective": l2, "device_type": "cpu", "verbosity": -1}, ds, 20)
    b2 = fb.train({"objective": "regression", "device_type": "cpu", "verbosity": -1, "boost_from_average": False}, fb.Dataset(X, y), 20)
    np.testing.assert_allclose(b1.predict(X), b2.predict(X), atol=1e-6)
    b3 = fb.train({"objective": "regression", "device_type": "cpu", "verbosity": -1}, fb.Dataset(X, y, free_raw_data=False), 10, init_model=b2)
    assert b3.num_trees() == 30
    assert np.mean((b3.predict(X) - y) ** 2) < np.mean((b2.predict(X) - y) ** 2)


def test_linear_tree_fits_piecewise_linear_target(tmp_path):
    """linear_tree=true: ridge regression on each leaf's path features; beats constant leaves on a
    piecewise-linear target, survives the text model round trip, validation scores equal predict()."""
    rng = np.random.default_rng(0)
    n = 8000

    def target(A):
        return np.where(A[:, 0] > 0, 2 * A[:, 1] + 1, -3 * A[:, 2]).astype(np.float32)

    X = rng.normal(size=(n, 5)).astype(np.float32)
    y = target(X) + 0.05 * rng.normal(size=n).astype(np.float32)
    Xv = rng.normal(size=(2000, 5)).astype(np.float32)
    Xv[::50, 1] = np.nan   # rows with a missing path feature fall back to the constant output
    yv = target(np.nan_to_num(Xv))
    mse = {}
    for lin in (False, True):
        p = {"objective": "regression", "num_leaves": 8, "learning_rate": 0.2, "linear_tree": lin, "linear_lambda": 0.01,
             "verbose": -1, "min_data_in_leaf": 20}
        ds = fb.Dataset(X, y, params=p)
        dv = fb.Dataset(Xv, yv, reference=ds)
        ev = {}
        b = fb.train(p, ds, 25, valid_sets=[dv], valid_names=["v"], callbacks=[fb.record_evaluation(ev)])
        pr = b.predict(Xv)
        mse[lin] = float(np.mean((pr - yv) ** 2))
        assert abs(ev["v"]["l2"][-1] - mse[lin]) < 1e-9
        if lin:
            s = b.model_to_string()
            assert "is_linear=1" in s and "leaf_coeff=" in s
            path = tmp_path / "lin.txt"
            b.save_model(str(path))
            assert np.array_equal(fb.Booster(model_file=str(path)).predict(Xv), pr)
    assert mse[True] < 0.3 * mse[False]


def _monotone_violations(bst, ncol, col, sign, rng, predict=None):
    """Largest decrease (increase for sign < 0) of the prediction along `col` with the other columns fixed."""
    base = rng.normal(size=(200, ncol)).astype(np.float32)
    grid = np.linspace(-3, 3, 41, dtype=np.float32)
    worst = 0.0
    prev = None
    for g in grid:
        A = base.copy()
        A[:, col] = g
        p = np.asarray((predict or bst.predict)(A), dtype=np.float64)
        if prev is not None:
            worst = max(worst, float(np.max(sign * (prev - p))))
        prev = p
    return worst


def test_monotone_constraints_hold_over_the_whole_tree():
    """A constrained feature's effect is monotone in every tree: each split orders its children and the
    children's output ranges are inherited by the whole subtree."""
    rng = np.random.default_rng(3)
    n = 6000
    X = rng.normal(size=(n, 4)).astype(np.float32)
    y = (np.sin(2 * X[:, 0]) + 0.5 * X[:, 0] - np.cos(2 * X[:, 1]) - 0.3 * X[:, 1] + X[:, 2] * X[:, 0] * 0.5
         + 0.1 * rng.normal(size=n)).astype(np.float32)
    p = {"objective": "regression", "num_leaves": 31, "learning_rate": 0.2, "verbose": -1, "min_data_in_leaf": 10,
         "monotone_constraints": [1, -1, 0, 0]}
    b = fb.train(p, fb.Dataset(X, y), 30)
    assert _monotone_violations(b, 4, 0, +1, rng) <= 1e-10
    assert _monotone_violations(b, 4, 1, -1, rng) <= 1e-10
    free = fb.train({**p, "monotone_constraints": [0, 0, 0, 0]}, fb.Dataset(X, y), 30)
    assert _monotone_violations(free, 4, 0, +1, rng) > 1e-3   # the target itself is not monotone


def test_monotone_intermediate_and_advanced_methods_are_monotone_and_less_constraining():
    """monotone_constraints_method=intermediate bounds a leaf by its neighbours' outputs instead of the split's mid
    point; advanced bounds each child, per threshold, by the neighbours that its own part of the cell touches. Both stay
    monotone everywhere and each fits the training data better than the one before (reference test:
    tests/python_package_test/test_engine.py test_monotone_constraints, every method)."""
    rng = np.random.default_rng(3)
    n = 6000
    X = rng.normal(size=(n, 4)).astype(np.float32)
    y = (np.sin(2 * X[:, 0]) + 0.5 * X[:, 0] - np.cos(2 * X[:, 1]) - 0.3 * X[:, 1] + X[:, 2] * X[:, 0] * 0.5
         + 0.1 * rng.normal(size=n)).astype(np.float32)
    for policy in ("level", "leaf"):
        loss = {}
        for method in ("basic", "intermediate", "advanced"):
            p = {"objective": "regression", "num_leaves": 31, "learning_rate": 0.2, "verbose": -1, "min_data_in_leaf": 10,
                 "monotone_constraints": [1, -1, 0, 0], "monotone_constraints_method": method, "grow_policy": policy}
            b = fb.train(p, fb.Dataset(X, y), 30)
            assert _monotone_violations(b, 4, 0, +1, rng) <= 1e-10
            assert _monotone_violations(b, 4, 1, -1, rng) <= 1e-10
            loss[method] = float(np.mean((b.predict(X) - y) ** 2))
        assert loss["advanced"] < loss["intermediate"] < loss["basic"]


def _branch_feature_sets(bst):
    """Feature set of every root-to-leaf path of every tree."""
    out = []

    def walk(node, feats):
        if "split_feature" not in node:
            out.append(frozenset(feats))
            return
        f = feats | {int(node["split_feature"])}
        walk(node["left_child"], f)
        walk(node["right_child"], f)

    for t in bst.dump_model()["tree_info"]:
        walk(t["tree_structure"], frozenset())
    return out


def test_interaction_constraints_and_bynode_sampling():
    rng = np.random.default_rng(5)
    n = 5000
    X = rng.normal(size=(n, 6)).astype(np.float32)
    y = (X[:, 0] * X[:, 1] + X[:, 2] * X[:, 3] + X[:, 4] + 0.1 * rng.normal(size=n)).astype(np.float32)
    p = {"objective": "regression", "num_leaves": 15, "verbose": -1, "min_data_in_leaf": 10,
         "interaction_constraints": "[0,1],[2,3,4]"}
    b = fb.train(p, fb.Dataset(X, y), 10)
    sets = _branch_feature_sets(b)
    assert len(sets) > 20
    for s in sets:
        assert s <= {0, 1} or s <= {2, 3, 4}, s      # feature 5 is in no set: never used
    # per-node sampling: still learns, and differs from the unsampled model
    q = {"objective": "regression", "num_leaves": 15, "verbose": -1, "min_data_in_leaf": 10, "feature_fraction_bynode": 0.5}
    b2 = fb.train(q, fb.Dataset(X, y), 10)
    b3 = fb.train({**q, "feature_fraction_bynode": 1.0}, fb.Dataset(X, y), 10)
    assert b2.model_to_string() != b3.model_to_string()
    assert float(np.mean((b2.predict(X) - y) ** 2)) < 0.7 * float(np.var(y))


def test_forced_splits_shape_the_top_of_every_tree(tmp_path):
    import json
    rng = np.random.default_rng(7)
    X = rng.normal(size=(4000, 5)).astype(np.float32)
    y = (X[:, 0] + 0.5 * X[:, 1] * X[:, 2] + 0.1 * rng.normal(size=4000)).astype(np.float32)
    forced = {"feature": 3, "threshold": 0.25, "left": {"feature": 4, "threshold": -0.5}, "right": {"feature": 1, "threshold": 0.0}}
    path = tmp_path / "forced.json"
    path.write_text(json.dumps(forced))
    for policy in ("level", "leaf"):
        p = {"objective": "regression", "num_leaves": 15, "verbose": -1, "min_data_in_leaf": 10, "grow_policy": policy,
             "forcedsplits_filename": str(path)}
        b = fb.train(p, fb.Dataset(X, y), 3)
        for t in b.dump_model()["tree_info"]:
            root = t["tree_structure"]
            assert root["split_feature"] == 3 and abs(root["threshold"] - 0.25) < 0.2
            assert root["left_child"]["split_feature"] == 4 and root["right_child"]["split_feature"] == 1
            assert t["num_leaves"] == 15
        assert float(np.mean((b.predict(X) - y) ** 2)) < float(np.var(y))


def test_cegb_split_penalty_makes_smaller_trees():
    rng = np.random.default_rng(2)
    X = rng.normal(size=(3000, 5)).astype(np.float32)
    y = (X[:, 0] + 0.3 * X[:, 1] + 0.3 * rng.normal(size=3000)).astype(np.float32)
    p = {"objective": "regression", "num_leaves": 31, "verbose": -1, "min_data_in_leaf": 5}
    free = fb.train(p, fb.Dataset(X, y), 3)
    taxed = fb.train({**p, "cegb_penalty_split": 0.05, "cegb_tradeoff": 1.0}, fb.Dataset(X, y), 3)
    leaves = lambda b: sum(t["num_leaves"] for t in b.dump_model()["tree_info"])
    assert leaves(free) == 93 and 3 < leaves(taxed) < leaves(free)


def test_reset_training_data_needs_aligned_bins():
    """Trees refer to rows by bin index, so continuing on a dataset that was binned on its own is refused;
    a dataset constructed against the original one (same bin mappers) is accepted and scores correctly."""
    X, y = make_binary(3000, 8)
    X2, y2 = make_binary(3000, 8, seed=7)
    train = fb.Dataset(X, y, params={"max_bin": 63})
    bst = fb.train({"objective": "binary", "device_type": "cpu", "verbosity": -1, "max_bin": 63}, train, 5, keep_training_booster=True)
    stranger = fb.Dataset(X2, y2, params={"max_bin": 15}).construct()   # own mappers, other bin count
    with pytest.raises(fb.FalcataError, match="bin mappers differ"):
        bst.update(train_set=stranger)
    aligned = fb.Dataset(X2, y2, reference=train)
    bst.update(train_set=aligned)
    # the replayed training scores are the model's real scores on the new rows (6 trees now; check via the metric)
    p = np.clip(bst.predict(X2), 1e-15, 1 - 1e-15)
    want = float(-np.mean(y2 * np.log(p) + (1 - y2) * np.log(1 - p)))
    got = [v for (_, name, v, _) in bst.eval_train() if name == "binary_logloss"][0]
    assert abs(got - want) < 1e-6


def test_reset_parameter_schedules():
    """List and callable schedules reach the booster before each round; wrong lengths and other types are refused."""
    rng = np.random.default_rng(3)
    X = rng.normal(size=(400, 5)); y = X[:, 0] * 2 + rng.normal(size=400) * 0.1
    seen = []

    def probe(env):
        seen.append(env.params.get("learning_rate"))
    probe.before_iteration = True; probe.order = 20
    params = {"objective": "regression", "num_leaves": 7, "verbosity": -1, "learning_rate": 0.5, "min_data_in_leaf": 5}
    b1 = fb.train(dict(params), fb.Dataset(X, y), 4, callbacks=[fb.reset_parameter(learning_rate=[0.5, 0.25, 0.125, 0.0625]), probe])
    assert seen == [0.5, 0.25, 0.125, 0.0625]
    b2 = fb.train(dict(params), fb.Dataset(X, y), 4, callbacks=[fb.reset_parameter(learning_rate=lambda i: 0.5 * 0.5 ** i)])
    assert np.allclose(b1.predict(X), b2.predict(X))
    b3 = fb.train(dict(params), fb.Dataset(X, y), 4)
    assert not np.allclose(b1.predict(X), b3.predict(X))
    with pytest.raises(ValueError):
        fb.train(dict(params), fb.Dataset(X, y), 4, callbacks=[fb.reset_parameter(learning_rate=[0.1, 0.2])])
    with pytest.raises(ValueError):
        fb.reset_parameter(learning_rate=0.1)


def test_auc_mu_matches_pairwise_definition():
    """auc_mu against a direct evaluation of its definition (all class pairs, all row pairs, ties one half), with the
    default partition weights, a custom matrix and row weights."""
    rng = np.random.default_rng(8)
    n, k = 300, 3
    X = rng.normal(size=(n, 5))
    y = np.argmax(X[:, :3] + 0.8 * rng.normal(size=(n, 3)), axis=1).astype(np.float64)
    w = rng.uniform(0.5, 2.0, size=n)

    def brute(raw, W, weights):
        tot = 0.0
        for i in range(k):
            for j in range(i + 1, k):
                v = W[i] - W[j]; t1 = v[i] - v[j]
                d = t1 * (raw @ v)
                a = np.where(y == i)[0]; b = np.where(y == j)[0]
                s = 0.0
                for p in a:
                    s += weights[p] * (np.sum(weights[b] * (d[b] < d[p] - 1e-15)) + 0.5 * np.sum(weights[b] * (np.abs(d[b] - d[p]) < 1e-15)))
                tot += s / (weights[a].sum() * weights[b].sum())
        return 2 * tot / (k * (k - 1))

    for weights, wm in [(None, None), (w, None), (None, [0, 1, 3, 2, 0, 1, 1, 4, 0])]:
        params = {"objective": "multiclass", "num_class": k, "metric": "auc_mu", "num_leaves": 7, "verbosity": -1, "min_data_in_leaf": 5}
        if wm is not None:
            params["auc_mu_weights"] = wm
        rec = {}
        ds = fb.Dataset(X, y, weight=weights)
        bst = fb.train(params, ds, 6, valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(rec)])
        raw = np.asarray(bst.predict(X, raw_score=True))
        W = np.ones((k, k)) - np.eye(k) if wm is None else np.asarray(wm, dtype=float).reshape(k, k)
        want = brute(raw, W, np.ones(n) if weights is None else weights)
        assert abs(rec["train"]["auc_mu"][-1] - want) < 1e-9
        assert rec["train"]["auc_mu"][-1] > 0.8


def test_cegb_per_feature_penalties_steer_feature_choice():
    """Coupled penalty: a feature is charged until the model first uses it, so an expensive twin of a cheap feature is
    never bought. Lazy penalty: charged per row not yet sent through the feature, which keeps a costly feature out
    unless it pays for itself."""
    rng = np.random.default_rng(13)
    n = 3000
    a = rng.normal(size=n); b = rng.normal(size=n)
    X = np.column_stack([a, a + 0.01 * rng.normal(size=n), b, rng.normal(size=n)])   # column 1 is a noisy twin of column 0
    y = a + 0.5 * b + 0.1 * rng.normal(size=n)
    base = {"objective": "regression", "num_leaves": 15, "verbosity": -1, "min_data_in_leaf": 10, "learning_rate": 0.2}
    free = fb.train(dict(base), fb.Dataset(X, y), 15)
    imp_free = free.feature_importance()
    assert imp_free[0] > 0 and imp_free[1] > 0                                          # without penalties both twins get used
    coupled = fb.train(dict(base, cegb_tradeoff=1.0, cegb_penalty_feature_coupled=[0.0, 1e6, 0.0, 0.0]), fb.Dataset(X, y), 15)
    imp = coupled.feature_importance()
    assert imp[1] == 0 and imp[0] > 0 and imp[2] > 0
    # a coupled price below the feature's worth is paid once: the feature is used afterwards like any other
    cheap = fb.train(dict(base, cegb_tradeoff=1.0, cegb_penalty_feature_coupled=[1.0, 1.0, 1.0, 1.0]), fb.Dataset(X, y), 15)
    assert cheap.feature_importance()[0] + cheap.feature_importance()[1] > 0 and cheap.feature_importance()[2] > 0
    lazy = fb.train(dict(base, cegb_tradeoff=1.0, cegb_penalty_feature_lazy=[0.0, 0.0, 1e3, 0.0]), fb.Dataset(X, y), 15)
    assert lazy.feature_importance()[2] == 0 and lazy.feature_importance()[0] > 0
    with pytest.raises(fb.FalcataError):
        fb.train(dict(base, cegb_penalty_feature_coupled=[1.0, 2.0]), fb.Dataset(X, y), 2)


def test_multi_regression_trains_one_tree_per_target():
    """objective=multi_regression: y is [rows, targets]; each round grows a tree per target; prediction is [rows, targets];
    each target's column equals a single-target L2 model trained alone on it; l2 is averaged over rows and targets."""
    rng = np.random.default_rng(17)
    n = 1200
    X = rng.normal(size=(n, 6))
    Y = np.column_stack([X[:, 0] + 0.1 * rng.normal(size=n), -2 * X[:, 1] + X[:, 2] + 5.0, np.sin(X[:, 3])])
    p = {"objective": "multi_regression", "num_class": 3, "num_leaves": 7, "verbosity": -1, "min_data_in_leaf": 5, "metric": "l2", "learning_rate": 0.3}
    rec = {}
    ds = fb.Dataset(X, Y)
    bst = fb.train(p, ds, 12, valid_sets=[ds], valid_names=["train"], callbacks=[fb.record_evaluation(rec)])
    assert bst.num_trees() == 36 and bst.num_model_per_iteration() == 3
    pred = np.asarray(bst.predict(X))
    assert pred.shape == (n, 3)
    for t in range(3):
        one = fb.train({"objective": "regression", "num_leaves": 7, "verbosity": -1, "min_data_in_leaf": 5, "learning_rate": 0.3}, fb.Dataset(X, Y[:, t]), 12)
        assert np.allclose(pred[:, t], one.predict(X), atol=1e-9)
    assert abs(rec["train"]["l2"][-1] - np.mean((pred - Y.astype(np.float32)) ** 2)) < 1e-7   # labels are kept in float32
    again = fb.Booster(model_str=bst.model_to_string())
    assert np.array_equal(np.asarray(again.predict(X)), pred)
    with pytest.raises(fb.FalcataError):
        fb.train(dict(p, num_class=2), fb.Dataset(X, Y), 2)          # three label columns for two targets
    # cross-validation subsets keep the targets together
    res = fb.cv(p, fb.Dataset(X, Y), num_boost_round=5, nfold=3, stratified=False, seed=1)
    key = [k for k in res if k.endswith("l2-mean")][0]
    assert res[key][-1] < res[key][0]


def test_more_than_255_bins_train_on_the_host_whatever_the_device():
    rng = np.random.default_rng(31)
    X = rng.normal(size=(6000, 4)); y = np.sin(3 * X[:, 0]) + 0.05 * rng.normal(size=6000)
    p = {"objective": "regression", "num_leaves": 63, "max_bin": 1023, "verbosity": -1, "min_data_in_leaf": 5, "min_data_in_bin": 1}
    b = fb.train(p, fb.Dataset(X, y, params={"max_bin": 1023, "min_data_in_bin": 1}), 10)
    fine = np.mean((b.predict(X) - y) ** 2)
    coarse = np.mean((fb.train(dict(p, max_bin=15), fb.Dataset(X, y, params={"max_bin": 15}), 10).predict(X) - y) ** 2)
    assert fine < coarse
    assert b.dump_model()["feature_infos"] is not None


def test_fixedpoint_error_feedback_and_robust_scale_switches():
    """Fixed-point quantization: the error feedback and the outlier-robust scale are plan switches that the host
    learner honours too; with both off the rounding is the plain one (a different model), and on balanced data the
    robust scale does not fire (same model with and without it)."""
    rng = np.random.default_rng(61)
    X = rng.normal(size=(5000, 8)); y = (X[:, 0] - X[:, 1] + 0.5 * rng.normal(size=5000) > 0).astype(np.float64)
    p = {"objective": "binary", "num_leaves": 15, "verbosity": -1, "quant_mode": "fixedpoint", "quant_bins": 16, "min_data_in_leaf": 10}
    body = lambda b: b.model_to_string().split("\nparameters:")[0]
    full = fb.train(dict(p), fb.Dataset(X, y), 10)
    no_gate = fb.train(dict(p, cuda_plan="auto,robust_scale:off"), fb.Dataset(X, y), 10)
    no_ef = fb.train(dict(p, cuda_plan="auto,quant_ef:off"), fb.Dataset(X, y), 10)
    assert body(full) == body(no_gate)          # balanced gradients: no gap, no re-anchoring
    assert body(full) != body(no_ef)            # the residuals change the rounding from the second round on
    exact = fb.train(dict(p, quant_mode="none"), fb.Dataset(X, y), 10)
    ll = lambda b: float(np.mean(np.where(y > 0, -np.log(b.predict(X)), -np.log(1 - b.predict(X)))))
    assert ll(full) <= ll(no_ef) + 0.01 and abs(ll(full) - ll(exact)) < 0.03


def test_monotone_penalty_keeps_constrained_features_out_of_the_top_of_the_tree():
    rng = np.random.default_rng(71)
    X = rng.normal(size=(4000, 3)); y = 3 * X[:, 0] + X[:, 1] + 0.1 * rng.normal(size=4000)
    base = {"objective": "regression", "num_leaves": 15, "verbosity": -1, "min_data_in_leaf": 10, "monotone_constraints": [1, 0, 0]}

    def root_feature(p):
        return fb.train(p, fb.Dataset(X, y), 1).dump_model()["tree_info"][0]["tree_structure"]["split_feature"]
    assert root_feature(dict(base)) == 0                               # the strongest feature splits the root
    assert root_feature(dict(base, monotone_penalty=2.0)) != 0          # its gain is wiped out at depths 0 and 1
    deep = fb.train(dict(base, monotone_penalty=2.0), fb.Dataset(X, y), 1)
    assert deep.feature_importance()[0] > 0                             # and comes back further down
    pr = deep.predict(np.column_stack([np.linspace(-2, 2, 50), np.zeros(50), np.zeros(50)]))
    assert np.all(np.diff(pr) >= -1e-12)


def test_vectorised_threshold_scan_equals_the_scalar_scan_bit_for_bit():
    """The host learner scans plain features (no L1, no output cap, no smoothing, no monotone range) with a vectorised
    gain pass. lambda_l1=1e-300 sends the same training through the scalar scan without changing a single value
    (|g| - 1e-300 rounds back to |g|), so the two models must be identical, digit for digit."""
    from util import model_body

    rng = np.random.default_rng(11)
    X = rng.normal(size=(5000, 9)).astype(np.float32)
    X[::11, 2] = np.nan                       # a feature with a missing bin takes the general scan in both runs
    y = (X[:, 0] * X[:, 1] + np.sin(3 * X[:, 3]) + 0.3 * rng.normal(size=5000) > 0).astype(np.float32)
    base = {"objective": "binary", "num_leaves": 31, "max_bin": 255, "verbosity": -1, "min_data_in_leaf": 5, "device_type": "cpu"}
    fast = fb.train(dict(base), fb.Dataset(X, y), 12)
    slow = fb.train(dict(base, lambda_l1=1e-300), fb.Dataset(X, y), 12)
    assert model_body(fast.model_to_string()) == model_body(slow.model_to_string())
    for threads in (1, 3):                    # and the result does not depend on the thread count
        again = fb.train(dict(base, num_threads=threads), fb.Dataset(X, y), 12)
        assert model_body(again.model_to_string()) == model_body(fast.model_to_string())


def test_histogram_pool_size_bounds_the_cached_histograms_without_changing_an_integer_model():
    """histogram_pool_size (MB) keeps only that many leaf histograms (least recently used dropped first); a leaf whose
    histogram is gone gets both children built from the data. Integer histograms make both routes exact, so the model
    is the same digit for digit; with real-valued bins the subtraction rounds differently and the predictions agree
    closely (reference: src/treelearner/feature_histogram.hpp HistogramPool)."""
    from util import model_body

    rng = np.random.default_rng(21)
    X = rng.normal(size=(6000, 12)).astype(np.float32)
    y = (X[:, 0] * X[:, 1] + X[:, 2] + 0.3 * rng.normal(size=6000) > 0).astype(np.float32)
    per_leaf_mb = 12 * 64 * 2 * 8 / (1 << 20)      # about 12 KB a leaf at max_bin 63
    for policy in ("level", "leaf"):
        base = {"objective": "binary", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "device_type": "cpu", "grow_policy": policy, "quant_mode": "fixedpoint", "quant_bins": 64}
        full = fb.train(dict(base), fb.Dataset(X, y), 8)
        tiny = fb.train(dict(base, histogram_pool_size=3 * per_leaf_mb), fb.Dataset(X, y), 8)   # three histograms at a time
        assert model_body(full.model_to_string()) == model_body(tiny.model_to_string())
    real = {"objective": "binary", "num_leaves": 31, "max_bin": 63, "verbosity": -1, "device_type": "cpu", "grow_policy": "leaf"}
    a = fb.train(dict(real), fb.Dataset(X, y), 8).predict(X)
    b = fb.train(dict(real, histogram_pool_size=3 * per_leaf_mb), fb.Dataset(X, y), 8).predict(X)
    assert np.max(np.abs(a - b)) < 1e-6


def test_host_learner_is_invariant_to_thread_count_and_histogram_pool():
    """Random small training jobs on the host learner: the model does not depend on the number of worker threads (below
    8192 rows the histogram of a bin adds its rows in row order whatever the thread count; the per-feature records are
    merged in a fixed order) nor, with integer histograms, on a histogram pool that holds a handful of leaves only."""
    from util import model_body

    rng = np.random.default_rng(123)
    for _ in range(6):
        n = int(rng.choice([800, 3000, 7000])); f = int(rng.choice([3, 9, 20]))
        X = rng.normal(size=(n, f)).astype(np.float32)
        if rng.random() < 0.5:
            X[rng.random(size=n) < 0.1, 0] = np.nan
        if rng.random() < 0.5:
            X[:, 1] = np.round(X[:, 1] * 2)
        y = (np.nan_to_num(X[:, 0]) * X[:, 1] + X[:, 2 % f] + 0.3 * rng.normal(size=n) > 0).astype(np.float32)
        p = {"objective": "binary", "num_leaves": int(rng.choice([7, 31, 63])), "max_bin": int(rng.choice([15, 63, 255])), "verbosity": -1, "device_type": "cpu",
             "min_data_in_leaf": int(rng.choice([1, 5, 20])), "grow_policy": str(rng.choice(["level", "leaf"])), "feature_fraction": float(rng.choice([1.0, 0.6])),
             "seed": int(rng.integers(100))}
        if rng.random() < 0.4:
            p["extra_trees"] = True
        if rng.random() < 0.4:
            p["feature_fraction_bynode"] = 0.7
        quant = dict(p, quant_mode="fixedpoint", quant_bins=64)
        base = model_body(fb.train(dict(quant, num_threads=8), fb.Dataset(X, y), 4).model_to_string())
        assert base == model_body(fb.train(dict(quant, num_threads=1), fb.Dataset(X, y), 4).model_to_string()), p
        assert base == model_body(fb.train(dict(quant, num_threads=8, histogram_pool_size=0.05), fb.Dataset(X, y), 4).model_to_string()), p
        real = dict(p, quant_mode="none")
        assert model_body(fb.train(dict(real, num_threads=8), fb.Dataset(X, y), 4).model_to_string()) == \
            model_body(fb.train(dict(real, num_threads=1), fb.Dataset(X, y), 4).model_to_string()), p


def test_quantized_training_keeps_monotone_and_interaction_constraints_on_the_host_learner():
    """The host learner combines quantized gradients with monotone constraints (every method; with the basic method the
    leaf renewal from the true gradients is clamped into the leaf's range) and with interaction constraints, given as a
    list of lists (reference: quantized training with constraints is refused on device_type=cuda only)."""
    rng = np.random.default_rng(3)
    n = 6000
    X = rng.normal(size=(n, 4)).astype(np.float32)
    y = (np.sin(2 * X[:, 0]) + 0.5 * X[:, 0] - np.cos(2 * X[:, 1]) - 0.3 * X[:, 1] + X[:, 2] * X[:, 0] * 0.5 + 0.1 * rng.normal(size=n)).astype(np.float32)
    for method, renew in (("basic", True), ("basic", False), ("intermediate", True), ("advanced", True)):
        p = {"objective": "regression", "num_leaves": 31, "learning_rate": 0.2, "verbose": -1, "min_data_in_leaf": 10, "monotone_constraints": [1, -1, 0, 0],
             "monotone_constraints_method": method, "quant_mode": "fixedpoint", "quant_bins": 16, "quant_train_renew_leaf": renew, "device_type": "cpu"}
        b = fb.train(p, fb.Dataset(X, y), 20)
        assert _monotone_violations(b, 4, 0, +1, rng) <= 1e-10 and _monotone_violations(b, 4, 1, -1, rng) <= 1e-10
        assert float(np.mean((b.predict(X) - y) ** 2)) < 0.6 * float(np.var(y))
    z = (X[:, 0] * X[:, 1] + X[:, 2] * X[:, 3] + X[:, 0] * X[:, 2] + 0.1 * rng.normal(size=n)).astype(np.float32)
    for quant in ("none", "fixedpoint", "stochastic"):
        p = {"objective": "regression", "num_leaves": 31, "verbose": -1, "interaction_constraints": [[0, 1], [2, 3]], "quant_mode": quant, "device_type": "cpu"}
        sets = _branch_feature_sets(fb.train(p, fb.Dataset(X, z), 10))
        assert all(s <= {0, 1} or s <= {2, 3} for s in sets), quant
