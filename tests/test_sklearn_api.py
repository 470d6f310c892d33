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
