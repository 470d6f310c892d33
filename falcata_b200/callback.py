"""Training callbacks: early stopping, evaluation logging / recording, parameter schedules.
Parity: python-package/falcata/callback.py (early_stopping, log_evaluation, record_evaluation,
reset_parameter and the CallbackEnv / EarlyStopException protocol)."""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

__all__ = ["EarlyStopException", "early_stopping", "log_evaluation", "record_evaluation", "reset_parameter", "CallbackEnv"]


class EarlyStopException(Exception):
    def __init__(self, best_iteration: int, best_score: List[Tuple[str, str, float, bool]]) -> None:
        super().__init__()
        self.best_iteration = best_iteration
        self.best_score = best_score


@dataclass
class CallbackEnv:
    model: Any
    params: Dict[str, Any]
    iteration: int
    begin_iteration: int
    end_iteration: int
    evaluation_result_list: Optional[List[Tuple]]


def _format_eval_result(value: Tuple, show_stdv: bool = True) -> str:
    if len(value) == 4:
        return f"{value[0]}'s {value[1]}: {value[2]:g}"
    if len(value) == 5:
        return f"{value[0]}'s {value[1]}: {value[2]:g} + {value[4]:g}" if show_stdv else f"{value[0]}'s {value[1]}: {value[2]:g}"
    raise ValueError("Wrong metric value")


def log_evaluation(period: int = 1, show_stdv: bool = True) -> Callable:
    def _callback(env: CallbackEnv) -> None:
        if period > 0 and env.evaluation_result_list and (env.iteration + 1) % period == 0:
            result = "\t".join(_format_eval_result(x, show_stdv) for x in env.evaluation_result_list)
            print(f"[{env.iteration + 1}]\t{result}", flush=True)

    _callback.order = 10  # type: ignore[attr-defined]
    return _callback


def record_evaluation(eval_result: Dict[str, Dict[str, List[Any]]]) -> Callable:
    if not isinstance(eval_result, dict):
        raise TypeError("eval_result should be a dictionary")

    def _init(env: CallbackEnv) -> None:
        eval_result.clear()
        for item in env.evaluation_result_list or []:
            data_name, eval_name = item[0], item[1]
            eval_result.setdefault(data_name, OrderedDict())
            if len(item) == 4:
                eval_result[data_name].setdefault(eval_name, [])
            else:
                eval_result[data_name].setdefault(f"{eval_name}-mean", [])
                eval_result[data_name].setdefault(f"{eval_name}-stdv", [])

    def _callback(env: CallbackEnv) -> None:
        if env.iteration == env.begin_iteration:
            _init(env)
        for item in env.evaluation_result_list or []:
            if len(item) == 4:
                eval_result.setdefault(item[0], OrderedDict()).setdefault(item[1], []).append(item[2])   # (the first evaluated iteration may come later)
            else:
                eval_result.setdefault(item[0], OrderedDict()).setdefault(f"{item[1]}-mean", []).append(item[2])
                eval_result[item[0]].setdefault(f"{item[1]}-stdv", []).append(item[4])

    _callback.order = 20  # type: ignore[attr-defined]
    return _callback


def reset_parameter(**kwargs: Union[list, Callable]) -> Callable:
    """Schedule parameters over the boosting rounds: each keyword maps a parameter name to a list (one value per
    round) or to a function of the round index (counted from the first round of this training call).
    Parity: python-package/falcata/callback.py (``reset_parameter``: runs before the iteration, order 10)."""
    schedules = dict(kwargs)
    for name, sched in schedules.items():
        if not isinstance(sched, list) and not callable(sched):
            raise ValueError("Only list and callable values are supported as a mapping from boosting round index to new parameter value.")

    def _value_at(name: str, sched: Union[list, Callable], step: int, n_rounds: int) -> Any:
        if callable(sched):
            return sched(step)
        if len(sched) != n_rounds:
            raise ValueError(f"Length of list {name!r} has to equal to 'num_boost_round'.")
        return sched[step]

    def _callback(env: CallbackEnv) -> None:
        step = env.iteration - env.begin_iteration
        n_rounds = env.end_iteration - env.begin_iteration
        changed = {}
        for name, sched in schedules.items():
            v = _value_at(name, sched, step, n_rounds)
            if name not in env.params or env.params[name] != v:
                changed[name] = v
        if not changed:
            return
        reset = getattr(env.model, "reset_parameter", None)
        if reset is not None:
            reset(changed)
        env.params.update(changed)

    _callback.before_iteration = True  # type: ignore[attr-defined]
    _callback.order = 10  # type: ignore[attr-defined]
    return _callback


def early_stopping(stopping_rounds: int, first_metric_only: bool = False, verbose: bool = True, min_delta: Union[float, List[float]] = 0.0,
                   min_iterations: int = 0) -> Callable:
    """``min_iterations``: a warm-up; iterations before it neither record a best score nor count towards stopping, so the best
    iteration is never below it."""
    if not isinstance(stopping_rounds, int) or stopping_rounds <= 0:
        raise ValueError(f"stopping_rounds should be an integer and greater than 0. got: {stopping_rounds}")
    if min_iterations < 0:
        raise ValueError("Early stopping min_iterations must be non-negative.")
    # "evals" counts the evaluations seen and "best_eval" the evaluation at which a score was best: with train(eval_freq=k)
    # only every k-th iteration is evaluated and stopping_rounds counts evaluations, not iterations
    state: Dict[str, Any] = {"enabled": True, "inited": False, "evals": 0, "best_eval": [], "best_score": [], "best_iter": [], "best_list": [], "cmp": [], "first_metric": ""}

    def _init(env: CallbackEnv) -> None:
        state["enabled"] = bool(env.evaluation_result_list)
        if not state["enabled"]:
            raise ValueError("For early stopping, at least one dataset and eval metric is required for evaluation")
        only_train = all(item[0] in ("training", getattr(env.model, "_train_data_name", "training")) for item in env.evaluation_result_list)
        if only_train and not hasattr(env.model, "cvfolds"):
            state["enabled"] = False
            return
        if verbose:
            print(f"Training until validation scores don't improve for {stopping_rounds} rounds", flush=True)
        n = len(env.evaluation_result_list)
        deltas = min_delta if isinstance(min_delta, list) else [min_delta] * n
        if len(deltas) < n:
            deltas = (deltas * n)[:n]
        state["best_score"] = []; state["best_iter"] = []; state["best_list"] = []; state["cmp"] = []; state["best_eval"] = []; state["evals"] = 0
        state["first_metric"] = env.evaluation_result_list[0][1].split(" ")[-1]
        for item, d in zip(env.evaluation_result_list, deltas):
            state["best_iter"].append(0); state["best_list"].append(None); state["best_eval"].append(0)
            if item[3]:
                state["best_score"].append(float("-inf")); state["cmp"].append(lambda a, b, d=d: a > b + d)
            else:
                state["best_score"].append(float("inf")); state["cmp"].append(lambda a, b, d=d: a < b - d)

    def _final_check(env: CallbackEnv, i: int) -> None:
        if env.iteration == env.end_iteration - 1:
            if verbose:
                best = "\t".join(_format_eval_result(x) for x in state["best_list"][i])
                print(f"Did not meet early stopping. Best iteration is:\n[{state['best_iter'][i] + 1}]\t{best}", flush=True)
            raise EarlyStopException(state["best_iter"][i], state["best_list"][i])

    def _callback(env: CallbackEnv) -> None:
        if env.iteration == env.begin_iteration:
            state["inited"] = False
        sparse_evals = int(getattr(env.model, "_eval_freq", 1) or 1) > 1
        if not env.evaluation_result_list and sparse_evals:
            return                                   # an iteration that train(eval_freq=k) did not evaluate
        if not state["inited"]:
            _init(env); state["inited"] = True
        if not state["enabled"]:
            return
        if env.iteration + 1 < min_iterations:
            return
        state["evals"] += 1
        for i, item in enumerate(env.evaluation_result_list):
            score = item[2]
            if state["best_list"][i] is None or state["cmp"][i](score, state["best_score"][i]):
                state["best_score"][i] = score; state["best_iter"][i] = env.iteration; state["best_list"][i] = env.evaluation_result_list; state["best_eval"][i] = state["evals"]
            metric_name = item[1].split(" ")[-1]
            if first_metric_only and state["first_metric"] != metric_name:
                continue
            if item[0] in ("training", getattr(env.model, "_train_data_name", "training")) and not hasattr(env.model, "cvfolds"):
                continue
            if state["evals"] - state["best_eval"][i] >= stopping_rounds:
                if verbose:
                    best = "\t".join(_format_eval_result(x) for x in state["best_list"][i])
                    print(f"Early stopping, best iteration is:\n[{state['best_iter'][i] + 1}]\t{best}", flush=True)
                raise EarlyStopException(state["best_iter"][i], state["best_list"][i])
            _final_check(env, i)

    _callback.order = 30  # type: ignore[attr-defined]
    return _callback
