"""Foreign gradient-boosting models as ordinary Boosters.

``from_xgboost`` reads an XGBoost ``gbtree`` model (a ``Booster``/sklearn wrapper, a JSON file, or the
parsed JSON dict); ``from_catboost`` reads a CatBoost model over numerical features (an object with
``save_model(..., format="json")``, a JSON file, or the parsed dict). Both emit the LightGBM-compatible
text model and load it with :class:`Booster`, so prediction (host and device), FALB serialisation and
``trees_to_dataframe`` work on the result.

What has to be reconciled, and how:

* XGBoost routes ``x < t`` left, this engine ``x <= t``. The threshold becomes the largest float32 below
  ``t``: no float32 value lies between the two, and XGBoost compares in float32.
* XGBoost's ``base_score`` lives in output space; it goes through the inverse link of the objective and
  becomes a constant first tree (one per class for multiclass).
* XGBoost numbers are float32: thresholds and leaf values are recovered through ``numpy.float32``.
* CatBoost trees are oblivious (one split per depth, ``value > border`` goes to the set bit): every level
  is expanded into ordinary binary nodes; ``scale`` and ``bias`` are folded into leaves / a constant tree.

Parity: python-package/falcata/importers.py (from_xgboost L259, from_catboost L478).
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from .basic import Booster

__all__ = ["from_xgboost", "from_catboost"]

_DEFAULT_LEFT = 2
_MISSING_NAN = 2 << 2


def _fmt(v: float) -> str:
    return repr(float(v))


class _TreeText:
    """Accumulates one binary tree in the text model's array layout."""

    def __init__(self) -> None:
        self.split_feature: List[int] = []
        self.threshold: List[float] = []
        self.decision_type: List[int] = []
        self.left: List[int] = []
        self.right: List[int] = []
        self.gain: List[float] = []
        self.internal_value: List[float] = []
        self.internal_count: List[int] = []
        self.leaf_value: List[float] = []
        self.leaf_count: List[int] = []

    def add_internal(self, feature: int, threshold: float, default_left: bool, gain: float = 0.0, count: int = 0) -> int:
        self.split_feature.append(int(feature)); self.threshold.append(float(threshold))
        self.decision_type.append((_DEFAULT_LEFT if default_left else 0) | _MISSING_NAN)
        self.left.append(0); self.right.append(0); self.gain.append(float(gain)); self.internal_value.append(0.0); self.internal_count.append(int(count))
        return len(self.split_feature) - 1

    def add_leaf(self, value: float, count: int = 0) -> int:
        self.leaf_value.append(float(value)); self.leaf_count.append(int(count))
        return ~(len(self.leaf_value) - 1)

    def text(self, index: int, shrinkage: float = 1.0) -> str:
        nl = len(self.leaf_value)
        j = lambda xs, f=str: " ".join(f(x) for x in xs)
        lines = [f"Tree={index}", f"num_leaves={nl}", "num_cat=0"]
        if nl > 1:
            lines += [f"split_feature={j(self.split_feature)}", f"split_gain={j(self.gain, _fmt)}", f"threshold={j(self.threshold, _fmt)}",
                      f"decision_type={j(self.decision_type)}", f"left_child={j(self.left)}", f"right_child={j(self.right)}"]
        lines.append(f"leaf_value={j(self.leaf_value, _fmt)}")
        if nl > 1:
            lines += [f"leaf_weight={j([0.0] * nl, _fmt)}", f"leaf_count={j(self.leaf_count)}", f"internal_value={j(self.internal_value, _fmt)}",
                      f"internal_weight={j([0.0] * (nl - 1), _fmt)}", f"internal_count={j(self.internal_count)}"]
        lines += ["is_linear=0", f"shrinkage={_fmt(shrinkage)}", "", ""]
        return "\n".join(lines)


def _constant_tree(index: int, value: float) -> str:
    t = _TreeText(); t.add_leaf(value)
    return t.text(index)


def _assemble(trees: Sequence[str], num_class: int, num_tree_per_iteration: int, objective: str, feature_names: Sequence[str]) -> Booster:
    header = ["tree", "version=v4", f"num_class={num_class}", f"num_tree_per_iteration={num_tree_per_iteration}", "label_index=0",
              f"max_feature_idx={len(feature_names) - 1}", f"objective={objective}", "feature_names=" + " ".join(feature_names),
              "feature_infos=" + " ".join(["none"] * len(feature_names)), "tree_sizes=" + " ".join(str(len(t.encode("utf-8"))) for t in trees), "", ""]
    text = "\n".join(header) + "".join(trees) + "end of trees\n\nfeature_importances:\n\nparameters:\n[boosting: gbdt]\n[objective: " + objective.split(" ")[0] + "]\n\nend of parameters\n\npandas_categorical:null\n"
    return Booster(model_str=text)


# ------------------------------------------------------------------ XGBoost ----
def _f32_below(t: float) -> float:
    """Largest float32 strictly below float32(t): ``x <= result`` is ``x < t`` for every float32 x."""
    return float(np.nextafter(np.float32(t), np.float32(-np.inf)))


def _xgb_dict(model: Any) -> Dict[str, Any]:
    if isinstance(model, dict):
        return model
    if isinstance(model, (str, Path)):
        return json.loads(Path(model).read_text())
    if hasattr(model, "get_booster"):
        model = model.get_booster()
    if hasattr(model, "save_raw"):
        return json.loads(bytes(model.save_raw(raw_format="json")).decode("utf-8"))
    raise TypeError("from_xgboost takes an xgboost Booster / sklearn model, a JSON model file or its parsed dict")


def _xgb_objective(name: str, num_class: int, base_score: float) -> Tuple[str, int, int, List[float]]:
    """-> (objective line, num_class, trees per iteration, raw-space base margin per class)."""
    if name in ("binary:logistic", "binary:logitraw", "reg:logistic"):
        p = min(max(base_score, 1e-12), 1 - 1e-12)
        return "binary sigmoid:1", 1, 1, [math.log(p / (1 - p)) if name != "binary:logitraw" else base_score]
    if name in ("multi:softprob", "multi:softmax"):
        return f"multiclass num_class:{num_class}", num_class, num_class, [base_score] * num_class
    if name in ("count:poisson", "reg:gamma", "reg:tweedie"):
        obj = {"count:poisson": "poisson", "reg:gamma": "gamma", "reg:tweedie": "tweedie"}[name]
        return obj, 1, 1, [math.log(max(base_score, 1e-12))]
    if name.startswith("rank:"):
        return "lambdarank", 1, 1, [base_score]
    if name in ("reg:squarederror", "reg:linear", "reg:squaredlogerror", "reg:pseudohubererror", "reg:absoluteerror"):
        return "regression", 1, 1, [base_score]
    raise ValueError(f"XGBoost objective {name!r} has no counterpart here")


def _xgb_tree(tree: Dict[str, Any], index: int) -> str:
    lefts, rights = tree["left_children"], tree["right_children"]
    feats, conds, dleft = tree["split_indices"], tree["split_conditions"], tree["default_left"]
    gains = tree.get("loss_changes", [0.0] * len(lefts)); covers = tree.get("sum_hessian", [0.0] * len(lefts))
    if any(int(t) != 0 for t in tree.get("split_type", [])):
        raise ValueError("XGBoost categorical splits are not supported by the importer")
    out = _TreeText()

    def emit(node: int) -> int:
        if lefts[node] == -1:
            return out.add_leaf(float(np.float32(conds[node])), int(covers[node]))
        me = out.add_internal(feats[node], _f32_below(conds[node]), bool(dleft[node]), float(np.float32(gains[node])), int(covers[node]))
        out.left[me] = emit(lefts[node]); out.right[me] = emit(rights[node])
        return me

    emit(0)
    return out.text(index)


def from_xgboost(model: Any, feature_names: Optional[List[str]] = None) -> Booster:
    """Convert an XGBoost gbtree model. Predictions agree with XGBoost's on float32 inputs."""
    raw = _xgb_dict(model)
    learner = raw["learner"]
    gb = learner["gradient_booster"]
    if gb.get("name", "gbtree") not in ("gbtree",):
        raise ValueError(f"only gbtree boosters can be imported, not {gb.get('name')!r}")
    lp = learner["learner_model_param"]
    num_class = max(1, int(lp.get("num_class", "0") or 0))
    nfeat = int(lp["num_feature"])
    bs = lp.get("base_score", "0.5")
    base = float(json.loads(bs)[0]) if isinstance(bs, str) and bs.strip().startswith("[") else float(bs)
    objective, nclass, per_iter, margins = _xgb_objective(learner["objective"]["name"], num_class, base)
    names = list(feature_names) if feature_names else (learner.get("feature_names") or [f"Column_{i}" for i in range(nfeat)])
    if len(names) != nfeat:
        raise ValueError(f"the model has {nfeat} features but {len(names)} names were given")
    trees_json = gb["model"]["trees"]; info = gb["model"].get("tree_info", [0] * len(trees_json))
    trees: List[str] = [_constant_tree(k, margins[k]) for k in range(per_iter)]
    # XGBoost stores trees round by round with the class in tree_info; the text model wants class-major rounds
    by_class: List[List[Dict[str, Any]]] = [[] for _ in range(per_iter)]
    for t, k in zip(trees_json, info):
        by_class[int(k) % per_iter].append(t)
    rounds = max(len(c) for c in by_class) if by_class else 0
    for r in range(rounds):
        for k in range(per_iter):
            idx = len(trees)
            trees.append(_xgb_tree(by_class[k][r], idx) if r < len(by_class[k]) else _constant_tree(idx, 0.0))
    return _assemble(trees, nclass, per_iter, objective, [str(n).replace(" ", "_") for n in names])


# ----------------------------------------------------------------- CatBoost ----
def _cb_dict(model: Any) -> Dict[str, Any]:
    if isinstance(model, dict):
        return model
    if isinstance(model, (str, Path)):
        return json.loads(Path(model).read_text())
    if hasattr(model, "save_model"):
        import os
        import tempfile

        with tempfile.TemporaryDirectory() as d:
            p = os.path.join(d, "m.json")
            model.save_model(p, format="json")
            return json.loads(Path(p).read_text())
    raise TypeError("from_catboost takes a CatBoost model, a JSON model file or its parsed dict")


def _cb_objective(raw: Dict[str, Any]) -> Tuple[str, int]:
    loss = str(raw.get("model_info", {}).get("params", {}).get("loss_function", {}).get("type", "RMSE"))
    if loss in ("Logloss", "CrossEntropy"):
        return "binary sigmoid:1", 1
    if loss in ("MultiClass", "MultiClassOneVsAll"):
        k = len(raw.get("model_info", {}).get("class_params", {}).get("class_names", [])) or 0
        return (f"multiclass num_class:{k}" if loss == "MultiClass" else f"multiclassova num_class:{k} sigmoid:1"), k
    if loss in ("Poisson", "Tweedie"):
        return loss.lower(), 1
    return "regression", 1


def _cb_tree(tree: Dict[str, Any], float_feature_of: Dict[int, int], dim: int, k: int, scale: float, index: int) -> str:
    """One oblivious tree, output dimension k of dim. Leaf index bit d is set when split d's test (value > border) holds."""
    splits = tree.get("splits", [])
    values = tree["leaf_values"]; weights = tree.get("leaf_weights", [0] * (len(values) // max(1, dim)))
    depth = len(splits)
    out = _TreeText()
    if depth == 0:
        out.add_leaf(scale * values[k])
        return out.text(index)
    for s in splits:
        if s.get("split_type", "FloatFeature") != "FloatFeature":
            raise ValueError("CatBoost models with categorical / text features are not supported by the importer")

    def emit(level: int, leaf_bits: int) -> int:
        # CatBoost applies splits[0] to the lowest bit; expand from the last split down so the tree is balanced either way
        if level < 0:
            return out.add_leaf(scale * values[leaf_bits * dim + k], int(weights[leaf_bits]) if leaf_bits < len(weights) else 0)
        s = splits[level]
        feat = float_feature_of[int(s["float_feature_index"])]
        # value > border -> bit set (right); value <= border -> left. NaN handling: CatBoost's default for numerical
        # features treats NaN as below every border ("Min"): it goes left.
        nan_left = str(s.get("nan_value_treatment", "AsIs")) != "AsTrue"
        me = out.add_internal(feat, float(np.float32(s["border"])), nan_left)
        out.left[me] = emit(level - 1, leaf_bits)
        out.right[me] = emit(level - 1, leaf_bits | (1 << level))
        return me

    emit(depth - 1, 0)
    return out.text(index)


def from_catboost(model: Any, feature_names: Optional[List[str]] = None) -> Booster:
    """Convert a CatBoost model over numerical features (oblivious trees)."""
    raw = _cb_dict(model)
    ff = raw.get("features_info", {}).get("float_features", [])
    if raw.get("features_info", {}).get("categorical_features"):
        raise ValueError("CatBoost models with categorical features are not supported by the importer")
    float_feature_of = {int(f.get("feature_index", i)): int(f.get("flat_feature_index", i)) for i, f in enumerate(ff)}
    nfeat = (max(float_feature_of.values()) + 1) if float_feature_of else 1
    names = list(feature_names) if feature_names else [str(f.get("feature_id") or f"Column_{float_feature_of[int(f.get('feature_index', i))]}") for i, f in enumerate(ff)]
    if len(names) != nfeat:
        names = [f"Column_{i}" for i in range(nfeat)]
    objective, k_decl = _cb_objective(raw)
    sb = raw.get("scale_and_bias", [1.0, [0.0]])
    scale = float(sb[0]); bias = sb[1] if isinstance(sb[1], list) else [float(sb[1])]
    obl = raw.get("oblivious_trees", [])
    dim = 1
    if obl:
        first = obl[0]
        dim = max(1, len(first["leaf_values"]) // (1 << len(first.get("splits", []))))
    if k_decl and k_decl != dim and dim > 1:
        objective = objective.replace(f"num_class:{k_decl}", f"num_class:{dim}")
    bias = (list(bias) + [0.0] * dim)[:dim]
    trees: List[str] = [_constant_tree(k, float(bias[k])) for k in range(dim)]
    for t in obl:
        for k in range(dim):
            trees.append(_cb_tree(t, float_feature_of, dim, k, scale, len(trees)))
    return _assemble(trees, dim if dim > 1 else 1, dim, objective, [str(n).replace(" ", "_") for n in names])
