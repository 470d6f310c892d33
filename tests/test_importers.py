"""Model importers against hand-built XGBoost / CatBoost JSON models and plain-Python evaluators of those formats."""
import math

import numpy as np

from falcata_b200.importers import from_catboost, from_xgboost


def _xgb_model():
    # tree 0: f0 < 0.5 ? (f1 < -1.25 ? 0.1 : -0.2) : 0.3 ; missing: node0 -> left, node1 -> right
    t0 = {"left_children": [1, 3, -1, -1, -1], "right_children": [2, 4, -1, -1, -1], "split_indices": [0, 1, 0, 0, 0],
          "split_conditions": [0.5, -1.25, 0.3, 0.1, -0.2], "default_left": [1, 0, 0, 0, 0], "loss_changes": [5.0, 2.0, 0, 0, 0],
          "sum_hessian": [100, 60, 40, 25, 35], "split_type": [0, 0, 0, 0, 0]}
    t1 = {"left_children": [1, -1, -1], "right_children": [2, -1, -1], "split_indices": [2, 0, 0], "split_conditions": [0.0, -0.05, 0.07],
          "default_left": [0, 0, 0], "loss_changes": [1.0, 0, 0], "sum_hessian": [100, 50, 50], "split_type": [0, 0, 0]}
    return {"learner": {"objective": {"name": "binary:logistic"}, "learner_model_param": {"num_class": "0", "num_feature": "3", "base_score": "2.5E-1"},
                        "gradient_booster": {"name": "gbtree", "model": {"trees": [t0, t1], "tree_info": [0, 0]}}}}


def _xgb_eval(model, X):
    lp = model["learner"]["learner_model_param"]
    base = float(lp["base_score"])
    out = np.full(len(X), math.log(base / (1 - base)))
    for t in model["learner"]["gradient_booster"]["model"]["trees"]:
        for i, x in enumerate(X):
            n = 0
            while t["left_children"][n] != -1:
                v = x[t["split_indices"][n]]
                if np.isnan(v):
                    n = t["left_children"][n] if t["default_left"][n] else t["right_children"][n]
                else:
                    n = t["left_children"][n] if np.float32(v) < np.float32(t["split_conditions"][n]) else t["right_children"][n]
            out[i] += np.float32(t["split_conditions"][n])
    return 1 / (1 + np.exp(-out))


def test_xgboost_import_routes_like_xgboost():
    m = _xgb_model()
    rng = np.random.RandomState(0)
    X = rng.randn(400, 3).astype(np.float32)
    X[:40, 0] = 0.5          # exactly on a threshold: x < t is false -> right
    X[40:80, 1] = -1.25
    X[80:100, 2] = 0.0
    X[100:130, 0] = np.nan
    X[130:160, 1] = np.nan
    X[160:170, 2] = np.nan
    bst = from_xgboost(m)
    np.testing.assert_allclose(bst.predict(X.astype(np.float64)), _xgb_eval(m, X), rtol=1e-6, atol=1e-7)
    assert bst.num_trees() == 3 and bst.num_feature() == 3
    # the result is an ordinary model: text round trip keeps the predictions
    import falcata_b200 as fb

    again = fb.Booster(model_str=bst.model_to_string())
    np.testing.assert_allclose(again.predict(X.astype(np.float64)), bst.predict(X.astype(np.float64)))


def _cb_model():
    # two oblivious trees of depth 2 over features 0 and 2; leaf index bit d = (x[f_d] > border_d)
    return {"features_info": {"float_features": [{"feature_index": 0, "flat_feature_index": 0}, {"feature_index": 1, "flat_feature_index": 1},
                                                  {"feature_index": 2, "flat_feature_index": 2}]},
            "model_info": {"params": {"loss_function": {"type": "RMSE"}}}, "scale_and_bias": [0.5, [1.25]],
            "oblivious_trees": [
                {"splits": [{"float_feature_index": 0, "border": 0.25, "split_type": "FloatFeature"}, {"float_feature_index": 2, "border": -0.5, "split_type": "FloatFeature"}],
                 "leaf_values": [1.0, 2.0, 3.0, 4.0], "leaf_weights": [10, 20, 30, 40]},
                {"splits": [{"float_feature_index": 1, "border": 0.0, "split_type": "FloatFeature"}], "leaf_values": [-1.0, 1.0], "leaf_weights": [50, 50]}]}


def _cb_eval(m, X):
    scale, bias = m["scale_and_bias"][0], m["scale_and_bias"][1][0]
    out = np.full(len(X), bias)
    for t in m["oblivious_trees"]:
        for i, x in enumerate(X):
            idx = 0
            for d, s in enumerate(t["splits"]):
                v = x[s["float_feature_index"]]
                if not np.isnan(v) and v > np.float32(s["border"]):
                    idx |= 1 << d
            out[i] += scale * t["leaf_values"][idx]
    return out


def test_catboost_import_expands_oblivious_trees():
    m = _cb_model()
    rng = np.random.RandomState(1)
    X = rng.randn(300, 3).astype(np.float32)
    X[:30, 0] = 0.25
    X[30:60, 2] = np.nan
    bst = from_catboost(m)
    np.testing.assert_allclose(bst.predict(X.astype(np.float64)), _cb_eval(m, X), rtol=1e-6, atol=1e-7)
