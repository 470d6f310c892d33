"""``train()`` and ``cv()``.
Parity: python-package/falcata/engine.py (train L109-369: alias handling, callbacks before/after
each iteration, early-stopping exception, best_iteration; cv + CVBooster)."""
from __future__ import annotations

import copy
from collections import defaultdict
from operator import attrgetter
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple, Union

import numpy as np

from . import callback
from .basic import _EARLY_STOP_ALIASES, _PARAM_ALIASES_NUM_ROUNDS, Booster, Dataset, FalcataError

__all__ = ["train", "cv", "CVBooster"]


def _pop_aliases(params: Dict[str, Any], aliases: Iterable[str], default: Any) -> Any:
    val = default
    for a in aliases:
        if a in params and params[a] is not None:
            val = params.pop(a)
    return val


def train(params: Dict[str, Any], train_set: Dataset, num_boost_round: int = 100, valid_sets: Optional[List[Dataset]] = None,
          valid_names: Optional[List[str]] = None, feval: Optional[Union[Callable, List[Callable]]] = None,
          init_model: Optional[Union[str, Booster]] = None, keep_training_booster: bool = False,
          callbacks: Optional[List[Callable]] = None, fobj: Optional[Callable] = None, eval_freq: int = 1) -> Booster:
    """Train a booster. ``params['objective']`` may be a callable ``(preds, train_data) -> (grad, hess)``.

    ``eval_freq``: the validation sets are evaluated every ``eval_freq`` iterations and on the last one; the callbacks
    that read the results (early stopping, logging, recording) do nothing on the other iterations, and early stopping's
    ``stopping_rounds`` then counts evaluations."""
    if int(eval_freq) < 1:
        raise ValueError(f"eval_freq must be >= 1, got {eval_freq}")
    eval_freq = int(eval_freq)
    params = copy.deepcopy(params) if params else {}
    if callable(params.get("objective")):
        fobj = params["objective"]; params["objective"] = "none"
    num_boost_round = int(_pop_aliases(params, _PARAM_ALIASES_NUM_ROUNDS, num_boost_round))
    if num_boost_round <= 0:
        raise ValueError("num_boost_round should be greater than zero.")
    early_rounds = _pop_aliases(params, _EARLY_STOP_ALIASES, None)
    first_metric_only = bool(params.get("first_metric_only", False))

    predictor = None
    if isinstance(init_model, (str, bytes)) or hasattr(init_model, "__fspath__"):
        predictor = Booster(model_file=init_model)
    elif isinstance(init_model, Booster):
        predictor = Booster(model_str=init_model.model_to_string(num_iteration=-1))
    init_iteration = predictor.current_iteration() if predictor is not None else 0
    if predictor is not None:
        train_set._set_predictor(predictor)

    train_set.params = {**train_set.params, **{k: v for k, v in params.items() if k not in train_set.params}}
    is_valid_contain_train = False
    train_data_name = "training"
    reduced_valid_sets: List[Dataset] = []
    name_valid_sets: List[str] = []
    if valid_sets is not None:
        if isinstance(valid_sets, Dataset):
            valid_sets = [valid_sets]
        if isinstance(valid_names, str):
            valid_names = [valid_names]
        for i, vd in enumerate(valid_sets):
            if vd is train_set:
                is_valid_contain_train = True
                if valid_names is not None:
                    train_data_name = valid_names[i]
                continue
            if predictor is not None:
                vd._set_predictor(predictor)
            if vd.reference is None:
                vd.set_reference(train_set)
            reduced_valid_sets.append(vd)
            name_valid_sets.append(valid_names[i] if valid_names is not None and len(valid_names) > i else f"valid_{i}")

    cbs = set(callbacks) if callbacks else set()
    if early_rounds is not None and int(early_rounds) > 0:
        cbs.add(callback.early_stopping(int(early_rounds), first_metric_only=first_metric_only, verbose=params.get("verbosity", 1) > 0,
                                        min_delta=params.get("early_stopping_min_delta", 0.0)))
    cbs_before = sorted((cb for cb in cbs if getattr(cb, "before_iteration", False)), key=attrgetter("order"))
    cbs_after = sorted((cb for cb in cbs if not getattr(cb, "before_iteration", False)), key=attrgetter("order"))

    from .basic import _tag
    with _tag("train: booster set-up (dataset construct included)"):
        booster = Booster(params=params, train_set=train_set)
    if is_valid_contain_train:
        booster.set_train_data_name(train_data_name)
    with _tag("train: add validation sets"):
        for vd, name in zip(reduced_valid_sets, name_valid_sets):
            booster.add_valid(vd, name)
    if predictor is not None:
        # continued training: the loaded trees come first in the final model
        import ctypes
        from .basic import _lib, _safe_call
        _safe_call(_lib().FB_BoosterMerge(booster._handle, predictor._handle))
    booster.best_iteration = 0
    booster._eval_freq = eval_freq

    evaluation_result_list: List[Tuple] = []
    for i in range(init_iteration, init_iteration + num_boost_round):
        for cb in cbs_before:
            cb(callback.CallbackEnv(model=booster, params=params, iteration=i, begin_iteration=init_iteration,
                                    end_iteration=init_iteration + num_boost_round, evaluation_result_list=None))
        with _tag("train: boosting rounds"):
            finished = booster.update(fobj=fobj)
        evaluation_result_list = []
        due = (i - init_iteration + 1) % eval_freq == 0 or i == init_iteration + num_boost_round - 1 or finished
        if (valid_sets is not None or feval is not None) and due:
            with _tag("train: metric evaluation"):
                if is_valid_contain_train:
                    evaluation_result_list.extend(booster.eval_train(feval))
                evaluation_result_list.extend(booster.eval_valid(feval))
        try:
            for cb in cbs_after:
                cb(callback.CallbackEnv(model=booster, params=params, iteration=i, begin_iteration=init_iteration,
                                        end_iteration=init_iteration + num_boost_round, evaluation_result_list=evaluation_result_list))
        except callback.EarlyStopException as es:
            booster.best_iteration = es.best_iteration + 1
            evaluation_result_list = es.best_score
            break
        if finished:
            break
    booster.best_score = defaultdict(dict)
    for item in evaluation_result_list or []:
        booster.best_score[item[0]][item[1]] = item[2]
    if not keep_training_booster:
        best_it, best_sc = booster.best_iteration, booster.best_score
        with _tag("train: copy of the model without training state"):
            model = Booster(model_str=booster.model_to_string(num_iteration=-1))
        model.best_iteration, model.best_score, model.params = best_it, best_sc, params
        return model
    return booster


class CVBooster:
    """Boosters of the cross-validation folds."""

    def __init__(self) -> None:
        self.boosters: List[Booster] = []
        self.best_iteration = -1
        self.cvfolds = True

    def _append(self, booster: Booster) -> None:
        self.boosters.append(booster)

    def __getattr__(self, name: str) -> Callable:
        def handler(*args: Any, **kwargs: Any) -> List[Any]:
            return [getattr(b, name)(*args, **kwargs) for b in self.boosters]

        return handler


def _make_n_folds(full: Dataset, folds: Any, nfold: int, params: Dict[str, Any], seed: int, stratified: bool, shuffle: bool):
    full.construct()
    n = full.num_data()
    if folds is not None:
        if hasattr(folds, "split"):
            group = full.get_group()
            gi = np.repeat(np.arange(len(group)), group) if group is not None else None
            folds = folds.split(X=np.empty(n), y=full.get_label(), groups=gi)
        return list(folds)
    group = full.get_group()
    rng = np.random.RandomState(seed)
    if group is not None:
        nq = len(group); q = rng.permutation(nq) if shuffle else np.arange(nq)
        bounds = np.concatenate([[0], np.cumsum(group)])
        out = []
        for k in range(nfold):
            tq = np.sort(q[k::nfold]); trq = np.sort(np.setdiff1d(q, tq))
            te = np.concatenate([np.arange(bounds[i], bounds[i + 1]) for i in tq]); tr = np.concatenate([np.arange(bounds[i], bounds[i + 1]) for i in trq])
            out.append((tr, te))
        return out
    idx = rng.permutation(n) if shuffle else np.arange(n)
    if stratified:
        y = full.get_label()
        order = np.argsort(y[idx], kind="stable"); idx = idx[order]
    out = []
    for k in range(nfold):
        te = np.sort(idx[k::nfold]); tr = np.sort(np.setdiff1d(idx, te))
        out.append((tr, te))
    return out


def _agg_cv_result(raw: List[List[Tuple]]) -> List[Tuple[str, str, float, bool, float]]:
    cvmap: Dict[Tuple[str, str], List[float]] = defaultdict(list)
    hib: Dict[Tuple[str, str], bool] = {}
    for one in raw:
        for item in one:
            key = (item[0], item[1]); cvmap[key].append(item[2]); hib[key] = item[3]
    return [(k[0], k[1], float(np.mean(v)), hib[k], float(np.std(v))) for k, v in cvmap.items()]


def cv(params: Dict[str, Any], train_set: Dataset, num_boost_round: int = 100, folds: Any = None, nfold: int = 5, stratified: bool = True,
       shuffle: bool = True, metrics: Optional[Union[str, List[str]]] = None, feval: Any = None, init_model: Any = None,
       callbacks: Optional[List[Callable]] = None, eval_train_metric: bool = False, return_cvbooster: bool = False, seed: int = 0,
       fobj: Optional[Callable] = None, fpreproc: Optional[Callable] = None) -> Dict[str, Any]:
    """K-fold cross-validation. Returns ``{'valid <metric>-mean': [...], 'valid <metric>-stdv': [...]}``.

    ``fpreproc(dtrain, dvalid, params) -> (dtrain, dvalid, params)`` is applied to every fold before its booster is made."""
    params = copy.deepcopy(params) if params else {}
    if callable(params.get("objective")):
        fobj = params["objective"]; params["objective"] = "none"
    num_boost_round = int(_pop_aliases(params, _PARAM_ALIASES_NUM_ROUNDS, num_boost_round))
    early_rounds = _pop_aliases(params, _EARLY_STOP_ALIASES, None)
    if metrics is not None:
        params["metric"] = metrics
    obj = str(params.get("objective", "regression"))
    if stratified and obj not in ("binary", "multiclass", "multiclassova", "softmax"):
        stratified = False
    train_set.params = {**train_set.params, **{k: v for k, v in params.items() if k not in train_set.params}}
    splits = _make_n_folds(train_set, folds, nfold, params, seed, stratified, shuffle)
    cvb = CVBooster()
    for tr, te in splits:
        dtrain = train_set.subset(np.asarray(tr)).construct(); dvalid = train_set.subset(np.asarray(te)).construct()
        fold_params = params
        if fpreproc is not None:
            dtrain, dvalid, fold_params = fpreproc(dtrain, dvalid, copy.deepcopy(params))
        b = Booster(fold_params, dtrain)
        if eval_train_metric:
            b.set_train_data_name("train")
        b.add_valid(dvalid, "valid")
        cvb._append(b)
    results: Dict[str, List[float]] = defaultdict(list)
    cbs = set(callbacks) if callbacks else set()
    if early_rounds is not None and int(early_rounds) > 0:
        cbs.add(callback.early_stopping(int(early_rounds), first_metric_only=bool(params.get("first_metric_only", False)), verbose=False))
    cbs_before = sorted((cb for cb in cbs if getattr(cb, "before_iteration", False)), key=attrgetter("order"))
    cbs_after = sorted((cb for cb in cbs if not getattr(cb, "before_iteration", False)), key=attrgetter("order"))
    for i in range(num_boost_round):
        for cb in cbs_before:
            cb(callback.CallbackEnv(model=cvb, params=params, iteration=i, begin_iteration=0, end_iteration=num_boost_round, evaluation_result_list=None))
        raw = []
        for b in cvb.boosters:
            b.update(fobj=fobj)
            one = []
            if eval_train_metric:
                one.extend(b.eval_train(feval))
            one.extend(b.eval_valid(feval))
            raw.append(one)
        res = _agg_cv_result(raw)
        for _, key, mean, _, std in [(r[0], f"{r[0]} {r[1]}", r[2], r[3], r[4]) for r in res]:
            results[f"{key}-mean"].append(mean); results[f"{key}-stdv"].append(std)
        try:
            for cb in cbs_after:
                cb(callback.CallbackEnv(model=cvb, params=params, iteration=i, begin_iteration=0, end_iteration=num_boost_round,
                                        evaluation_result_list=[(r[0], f"{r[0]} {r[1]}" if False else r[1], r[2], r[3], r[4]) for r in res]))
        except callback.EarlyStopException as es:
            cvb.best_iteration = es.best_iteration + 1
            for b in cvb.boosters:
                b.best_iteration = cvb.best_iteration
            for k in results:
                results[k] = results[k][: cvb.best_iteration]
            break
    out: Dict[str, Any] = dict(results)
    if return_cvbooster:
        out["cvbooster"] = cvb
    return out
