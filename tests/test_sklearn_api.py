"""sklearn-style estimators and the ``falcata`` compatibility import."""
import numpy as np

from util import make_binary, make_multiclass, make_ranking, make_regression


def test_classifier_regressor_ranker():
    import falcata as fl

    X, y = make_binary(4000, 10)
    clf = fl.LGBMClassifier(n_estimators=30, num_leaves=15, device_type="cpu").fit(X[:3000], y[:3000], eval_set=[(X[3000:], y[3000:])], eval_metric="auc")
    assert (clf.predict(X[3000:]) == y[3000:]).mean() > 0.85
    proba = clf.predict_proba(X[3000:])
    assert proba.shape == (1000, 2) and np.allclose(proba.sum(1), 1)
    assert "auc" in clf.evals_result_["valid_0"] and clf.feature_importances_.sum() > 0 and clf.n_features_ == 10
    Xm, ym = make_multiclass(3000, 8, 3)
    cm = fl.FalcataClassifier(n_estimators=20, device_type="cpu").fit(Xm, ym)
    assert cm.predict_proba(Xm).shape == (3000, 3) and (cm.predict(Xm) == ym).mean() > 0.7
    Xr, yr = make_regression(3000, 6)
    reg = fl.LGBMRegressor(n_estimators=40, device_type="cpu").fit(Xr, yr)
    assert np.mean((reg.predict(Xr) - yr) ** 2) < 0.3 * np.var(yr)
    Xq, yq, g = make_ranking(100, 20, 8)
    rk = fl.LGBMRanker(n_estimators=10, min_child_samples=5, device_type="cpu").fit(Xq, yq, group=g)
    assert rk.predict(Xq).shape == (2000,)


def test_fit_takes_eval_X_eval_y_and_early_stopping_has_a_warm_up():
    import falcata_b200 as fb

    rng = np.random.default_rng(1)
    X = rng.normal(size=(2500, 6)); y = (X[:, 0] + X[:, 1] * X[:, 2] + rng.normal(size=2500) > 0).astype(int)
    clf = fb.FalcataClassifier(n_estimators=60, learning_rate=0.3, verbosity=-1, device_type="cpu")
    clf.fit(X[:2000], y[:2000], eval_X=X[2000:], eval_y=y[2000:], callbacks=[fb.early_stopping(3, verbose=False, min_iterations=25)])
    assert clf.best_iteration_ >= 25 and "valid_0" in clf.evals_result_
    both = fb.FalcataClassifier(n_estimators=5, verbosity=-1, device_type="cpu")
    both.fit(X[:2000], y[:2000], eval_X=(X[2000:2200], X[2200:]), eval_y=(y[2000:2200], y[2200:]), eval_class_weight=[{0: 1.0, 1: 3.0}, None])
    assert set(both.evals_result_) == {"valid_0", "valid_1"}
    import pytest

    with pytest.raises(ValueError):
        both.fit(X[:2000], y[:2000], eval_X=X[2000:])
    with pytest.raises(ValueError):
        both.fit(X[:2000], y[:2000], eval_X=X[2000:], eval_y=y[2000:], eval_set=[(X[2000:], y[2000:])])
