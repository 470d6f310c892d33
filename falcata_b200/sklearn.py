"""scikit-learn style estimators.
Parity: python-package/falcata/sklearn.py (LGBMModel / Classifier / Regressor / Ranker and the
Falcata-named aliases): constructor parameters, fit(eval_set, eval_metric, callbacks, init_model),
predict / predict_proba, best_iteration_, evals_result_, feature_importances_."""
from __future__ import annotations

import copy
from typing import Any, Callable, Dict, List, Optional, Union

import numpy as np

from .basic import Booster, Dataset
from .callback import record_evaluation
from .engine import train

try:
    from sklearn.base import BaseEstimator, ClassifierMixin, RegressorMixin
    from sklearn.preprocessing import LabelEncoder

    _SK = True
except ImportError:  # pragma: no cover
    BaseEstimator = object  # type: ignore

    class ClassifierMixin:  # type: ignore
        pass

    class RegressorMixin:  # type: ignore
        pass

    LabelEncoder = None  # type: ignore
    _SK = False

__all__ = ["LGBMModel", "LGBMClassifier", "LGBMRegressor", "LGBMRanker", "FalcataModel", "FalcataClassifier", "FalcataRegressor", "FalcataRanker"]


def _positional_arity(func: Callable) -> int:
    import inspect

    try:
        params = inspect.signature(func).parameters.values()
    except (TypeError, ValueError):
        return 2
    return sum(1 for q in params if q.kind in (q.POSITIONAL_ONLY, q.POSITIONAL_OR_KEYWORD) and q.default is q.empty)


class _ObjectiveFunctionWrapper:
    """Adapts an sklearn-style objective ``f(y_true, y_pred[, weight[, group]]) -> (grad, hess)`` to the training
    loop's ``fobj(preds, dataset)``. With two arguments the returned gradients are multiplied by the sample weights
    here; with three or four the function gets the weights (and query sizes) and applies them itself.
    Parity: python-package/falcata/sklearn.py (_ObjectiveFunctionWrapper)."""

    def __init__(self, func: Callable) -> None:
        self.func = func
        self.arity = _positional_arity(func)
        if self.arity not in (2, 3, 4):
            raise TypeError(f"Self-defined objective function should have 2, 3 or 4 arguments, got {self.arity}")

    def __call__(self, preds: Any, dataset: Dataset) -> Any:
        labels = dataset.get_label()
        weight = dataset.get_weight()
        if self.arity == 2:
            grad, hess = self.func(labels, preds)
            if weight is not None:
                w = np.asarray(weight, dtype=np.float64)
                grad = np.asarray(grad, dtype=np.float64); hess = np.asarray(hess, dtype=np.float64)
                if grad.ndim == 2:      # [rows, classes]
                    w = w[:, None]
                grad = grad * w; hess = hess * w
            return grad, hess
        if self.arity == 3:
            return self.func(labels, preds, weight)
        return self.func(labels, preds, weight, dataset.get_group())


class _EvalFunctionWrapper:
    """Adapts an sklearn-style metric ``f(y_true, y_pred[, weight[, group]]) -> (name, value, higher_is_better)`` (or a
    list of such triples) to the training loop's ``feval(preds, dataset)``.
    Parity: python-package/falcata/sklearn.py (_EvalFunctionWrapper)."""

    def __init__(self, func: Callable) -> None:
        self.func = func
        self.arity = _positional_arity(func)
        if self.arity not in (2, 3, 4):
            raise TypeError(f"Self-defined eval function should have 2, 3 or 4 arguments, got {self.arity}")

    def __call__(self, preds: Any, dataset: Dataset) -> Any:
        labels = dataset.get_label()
        if self.arity == 2:
            return self.func(labels, preds)
        if self.arity == 3:
            return self.func(labels, preds, dataset.get_weight())
        return self.func(labels, preds, dataset.get_weight(), dataset.get_group())


class LGBMModel(BaseEstimator):
    def __init__(self, boosting_type: str = "gbdt", num_leaves: int = 31, max_depth: int = -1, learning_rate: float = 0.1, n_estimators: int = 100,
                 subsample_for_bin: int = 200000, objective: Optional[Union[str, Callable]] = None, class_weight: Any = None, min_split_gain: float = 0.0,
                 min_child_weight: float = 1e-3, min_child_samples: int = 20, subsample: float = 1.0, subsample_freq: int = 0, colsample_bytree: float = 1.0,
                 reg_alpha: float = 0.0, reg_lambda: float = 0.0, random_state: Optional[int] = None, n_jobs: Optional[int] = None,
                 importance_type: str = "split", device_type: Optional[str] = None, **kwargs: Any) -> None:
        self.boosting_type = boosting_type; self.num_leaves = num_leaves; self.max_depth = max_depth; self.learning_rate = learning_rate
        self.n_estimators = n_estimators; self.subsample_for_bin = subsample_for_bin; self.objective = objective; self.class_weight = class_weight
        self.min_split_gain = min_split_gain; self.min_child_weight = min_child_weight; self.min_child_samples = min_child_samples
        self.subsample = subsample; self.subsample_freq = subsample_freq; self.colsample_bytree = colsample_bytree; self.reg_alpha = reg_alpha
        self.reg_lambda = reg_lambda; self.random_state = random_state; self.n_jobs = n_jobs; self.importance_type = importance_type
        self.device_type = device_type
        self._other_params: Dict[str, Any] = {}
        self._Booster: Optional[Booster] = None
        self._evals_result: Dict[str, Any] = {}
        self._best_iteration = -1
        self._best_score: Dict[str, Any] = {}
        self._n_features = -1
        self._n_classes = -1
        self._objective = objective
        self.set_params(**kwargs)

    def get_params(self, deep: bool = True) -> Dict[str, Any]:
        params = super().get_params(deep=deep) if _SK else {k: v for k, v in self.__dict__.items() if not k.startswith("_")}
        params.update(self._other_params)
        return params

    def set_params(self, **params: Any) -> "LGBMModel":
        for key, value in params.items():
            setattr(self, key, value)
            if hasattr(self, f"_{key}"):
                setattr(self, f"_{key}", value)
            if key not in self.__init__.__code__.co_varnames:  # type: ignore[misc]
                self._other_params[key] = value
        return self

    def _default_objective(self) -> str:
        return "regression"

    def _process_params(self) -> Dict[str, Any]:
        p = self.get_params()
        p.pop("importance_type", None); p.pop("n_estimators", None); p.pop("class_weight", None)
        if p.get("device_type") is None:
            p.pop("device_type", None)
        obj = p.pop("objective", None)
        self._fobj = _ObjectiveFunctionWrapper(obj) if callable(obj) else None
        p["objective"] = "none" if callable(obj) else (obj or self._default_objective())
        alias = {"boosting_type": "boosting", "min_split_gain": "min_gain_to_split", "min_child_weight": "min_sum_hessian_in_leaf", "min_child_samples": "min_data_in_leaf",
                 "subsample": "bagging_fraction", "subsample_freq": "bagging_freq", "colsample_bytree": "feature_fraction", "reg_alpha": "lambda_l1", "reg_lambda": "lambda_l2",
                 "subsample_for_bin": "bin_construct_sample_cnt", "random_state": "seed", "n_jobs": "num_threads"}
        out = {}
        for k, v in p.items():
            if v is None:
                continue
            out[alias.get(k, k)] = v
        out.setdefault("verbosity", -1)
        return out

    def fit(self, X: Any, y: Any, sample_weight: Any = None, init_score: Any = None, group: Any = None, eval_set: Any = None, eval_names: Any = None,
            eval_sample_weight: Any = None, eval_init_score: Any = None, eval_group: Any = None, eval_metric: Any = None, feature_name: Any = "auto",
            categorical_feature: Any = "auto", callbacks: Optional[List[Callable]] = None, init_model: Any = None, eval_X: Any = None, eval_y: Any = None,
            eval_class_weight: Any = None) -> "LGBMModel":
        # eval_X / eval_y (one pair or tuples of the same length) are the newer spelling of eval_set
        if eval_X is not None or eval_y is not None:
            if eval_set is not None:
                raise ValueError("Specify either 'eval_set' or 'eval_X' and 'eval_y', but not both.")
            if (eval_X is None) != (eval_y is None):
                raise ValueError("You must specify eval_X and eval_y, not just one of them.")
            if isinstance(eval_X, tuple) != isinstance(eval_y, tuple) or (isinstance(eval_X, tuple) and len(eval_X) != len(eval_y)):
                raise ValueError("If eval_X is a tuple, eval_y must be a tuple of the same length, and vice versa.")
            eval_set = list(zip(eval_X, eval_y)) if isinstance(eval_X, tuple) else [(eval_X, eval_y)]
        if eval_class_weight is not None and eval_set is not None:
            # per validation set a class -> weight mapping (or "balanced"): multiplied into that set's sample weights
            weights = list(eval_sample_weight) if eval_sample_weight is not None else [None] * len(eval_set)
            for i, (cw, (_, ey)) in enumerate(zip(eval_class_weight, eval_set)):
                if cw is None:
                    continue
                ey = np.asarray(ey).reshape(-1)
                classes, enc = np.unique(ey, return_inverse=True)
                w = len(ey) / (len(classes) * np.bincount(enc)) if cw == "balanced" else np.array([cw.get(c, 1.0) for c in classes])
                weights[i] = w[enc] if weights[i] is None else w[enc] * np.asarray(weights[i], dtype=np.float64)
            eval_sample_weight = weights
        params = self._process_params()
        if self._n_classes > 2 and params["objective"] in ("binary", "multiclass", "multiclassova"):
            params["num_class"] = self._n_classes
        feval = None
        if eval_metric is not None:
            metrics = eval_metric if isinstance(eval_metric, (list, tuple)) else [eval_metric]
            names = [m for m in metrics if isinstance(m, str)]
            fevals = [m for m in metrics if callable(m)]
            if names:
                params["metric"] = ",".join(names)
            if fevals:
                feval = [_EvalFunctionWrapper(f) for f in fevals]
        train_set = Dataset(X, label=y, weight=sample_weight, group=group, init_score=init_score, feature_name=feature_name,
                            categorical_feature=categorical_feature, params={k: params[k] for k in ("max_bin", "bin_construct_sample_cnt", "min_data_in_leaf") if k in params})
        valid_sets: List[Dataset] = []
        if eval_set is not None:
            if isinstance(eval_set, tuple):
                eval_set = [eval_set]
            for i, (vx, vy) in enumerate(eval_set):
                if vx is X and vy is y:
                    valid_sets.append(train_set)
                    continue
                vw = eval_sample_weight[i] if eval_sample_weight is not None else None
                vg = eval_group[i] if eval_group is not None else None
                vi = eval_init_score[i] if eval_init_score is not None else None
                valid_sets.append(train_set.create_valid(vx, label=self._encode_y(vy), weight=vw, group=vg, init_score=vi))
        self._evals_result = {}
        cbs = list(callbacks) if callbacks else []
        cbs.append(record_evaluation(self._evals_result))
        if isinstance(init_model, LGBMModel):
            init_model = init_model.booster_
        self._Booster = train(params, train_set, num_boost_round=self.n_estimators, valid_sets=valid_sets or None, valid_names=eval_names, feval=feval,
                              init_model=init_model, callbacks=cbs, fobj=self._fobj)
        self._n_features = self._Booster.num_feature()
        self._best_iteration = self._Booster.best_iteration
        self._best_score = self._Booster.best_score
        return self

    def __sklearn_is_fitted__(self) -> bool:
        return getattr(self, "_Booster", None) is not None

    def _more_tags(self) -> Dict[str, Any]:
        return {"allow_nan": True, "X_types": ["2darray", "sparse", "1dlabels"],
                "_xfail_checks": {"check_no_attributes_set_in_init": "the constructor keeps **kwargs for pass-through parameters"}}

    def __sklearn_tags__(self) -> Any:
        tags = super().__sklearn_tags__()
        tags.input_tags.allow_nan = True
        tags.input_tags.sparse = True
        return tags

    def _encode_y(self, y: Any) -> Any:
        return y

    def predict(self, X: Any, raw_score: bool = False, start_iteration: int = 0, num_iteration: Optional[int] = None, pred_leaf: bool = False,
                pred_contrib: bool = False, **kwargs: Any) -> Any:
        if self._Booster is None:
            raise RuntimeError("Estimator not fitted, call fit before exploiting the model.")
        return self._Booster.predict(X, raw_score=raw_score, start_iteration=start_iteration, num_iteration=num_iteration, pred_leaf=pred_leaf,
                                     pred_contrib=pred_contrib, **kwargs)

    @property
    def booster_(self) -> Booster:
        if self._Booster is None:
            raise RuntimeError("No booster found. Need to call fit beforehand.")
        return self._Booster

    @property
    def best_iteration_(self) -> int:
        return self._best_iteration

    @property
    def best_score_(self) -> Dict[str, Any]:
        return self._best_score

    @property
    def evals_result_(self) -> Dict[str, Any]:
        return self._evals_result

    @property
    def n_features_(self) -> int:
        return self._n_features

    @property
    def n_features_in_(self) -> int:
        return self._n_features

    @property
    def feature_importances_(self) -> np.ndarray:
        return self.booster_.feature_importance(importance_type=self.importance_type)

    @property
    def feature_name_(self) -> List[str]:
        return self.booster_.feature_name()

    @property
    def n_estimators_(self) -> int:
        """Boosting rounds actually trained (python-package/falcata/sklearn.py: n_estimators_)."""
        return self.booster_.current_iteration()

    @property
    def n_iter_(self) -> int:
        return self.booster_.current_iteration()

    @property
    def feature_names_in_(self) -> np.ndarray:
        return np.array(self.feature_name_)

    @property
    def objective_(self) -> Any:
        return self._objective or self._default_objective()


class LGBMRegressor(RegressorMixin, LGBMModel):
    def _default_objective(self) -> str:
        return "regression"


class LGBMClassifier(ClassifierMixin, LGBMModel):
    def _default_objective(self) -> str:
        return "binary" if self._n_classes <= 2 else "multiclass"

    def fit(self, X: Any, y: Any, **kwargs: Any) -> "LGBMClassifier":  # type: ignore[override]
        y = np.asarray(y.detach().cpu().numpy() if hasattr(y, "detach") else y).reshape(-1)
        self._classes, enc = np.unique(y, return_inverse=True)
        self._n_classes = len(self._classes)
        if self.class_weight is not None:
            # class weights multiply whatever sample weights were given
            if self.class_weight == "balanced":
                cw = len(y) / (self._n_classes * np.bincount(enc))
            else:
                cw = np.array([self.class_weight.get(c, 1.0) for c in self._classes])
            given = kwargs.get("sample_weight")
            kwargs["sample_weight"] = cw[enc] if given is None else cw[enc] * np.asarray(given, dtype=np.float64)
        super().fit(X, enc.astype(np.float32), **kwargs)
        return self

    def _encode_y(self, y: Any) -> Any:
        y = np.asarray(y).reshape(-1)
        lut = {c: i for i, c in enumerate(self._classes)}
        return np.array([lut[v] for v in y], dtype=np.float32)

    @property
    def classes_(self) -> np.ndarray:
        return self._classes

    @property
    def n_classes_(self) -> int:
        return self._n_classes

    def predict_proba(self, X: Any, raw_score: bool = False, start_iteration: int = 0, num_iteration: Optional[int] = None, pred_leaf: bool = False,
                      pred_contrib: bool = False, **kwargs: Any) -> Any:
        res = super().predict(X, raw_score, start_iteration, num_iteration, pred_leaf, pred_contrib, **kwargs)
        if hasattr(res, "is_cuda"):
            res = res.detach().cpu().numpy()
        if callable(self._objective) or raw_score or pred_leaf or pred_contrib:
            return res
        if self._n_classes > 2:
            return res
        return np.vstack((1.0 - res, res)).T

    def decision_function(self, X: Any, *, start_iteration: int = 0, num_iteration: Optional[int] = None, **kwargs: Any) -> Any:
        """Raw margin of every sample (python-package/falcata/sklearn.py: FalcataClassifier.decision_function)."""
        return self.predict_proba(X, raw_score=True, start_iteration=start_iteration, num_iteration=num_iteration, **kwargs)

    def predict(self, X: Any, raw_score: bool = False, start_iteration: int = 0, num_iteration: Optional[int] = None, pred_leaf: bool = False,
                pred_contrib: bool = False, **kwargs: Any) -> Any:
        res = self.predict_proba(X, raw_score, start_iteration, num_iteration, pred_leaf, pred_contrib, **kwargs)
        if callable(self._objective) or raw_score or pred_leaf or pred_contrib:
            return res
        return self._classes[np.argmax(res, axis=1)]


class LGBMRanker(LGBMModel):
    def _default_objective(self) -> str:
        return "lambdarank"

    def fit(self, X: Any, y: Any, group: Any = None, eval_at: Any = (1, 2, 3, 4, 5), **kwargs: Any) -> "LGBMRanker":  # type: ignore[override]
        if group is None:
            raise ValueError("Should set group for ranking task")
        if kwargs.get("eval_set") is not None and kwargs.get("eval_group") is None:
            raise ValueError("Eval_group cannot be None when eval_set is not None")
        self._other_params["eval_at"] = ",".join(str(int(k)) for k in eval_at)
        super().fit(X, y, group=group, **kwargs)
        return self


FalcataModel = LGBMModel
FalcataClassifier = LGBMClassifier
FalcataRegressor = LGBMRegressor
FalcataRanker = LGBMRanker
