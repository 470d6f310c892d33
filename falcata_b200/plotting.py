"""Host-side plots: feature importance, split-value histograms, metric curves and tree diagrams.

matplotlib and graphviz are optional and imported only when a plot is drawn. The data behind every plot is
available without them: :func:`importance_table`, :func:`split_value_histogram`, :func:`metric_curves` and
:func:`tree_to_dot` (DOT source as plain text).

Parity: python-package/falcata/plotting.py (plot_importance L37, plot_split_value_histogram L176,
plot_metric L294, create_tree_digraph L623, plot_tree L749).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple, Union

import numpy as np

from .basic import Booster

__all__ = ["plot_importance", "plot_split_value_histogram", "plot_metric", "create_tree_digraph", "plot_tree", "importance_table",
           "split_value_histogram", "metric_curves", "tree_to_dot"]


def _booster_of(obj: Any) -> Booster:
    if isinstance(obj, Booster):
        return obj
    if hasattr(obj, "booster_"):
        return obj.booster_
    raise TypeError("booster must be a Booster or a fitted estimator")


def _axes(ax: Any, figsize: Optional[Tuple[float, float]], dpi: Optional[int]) -> Any:
    try:
        import matplotlib.pyplot as plt
    except ImportError as e:  # pragma: no cover - optional dependency
        raise ImportError("matplotlib is needed for plotting") from e
    if ax is None:
        _, ax = plt.subplots(1, 1, figsize=figsize, dpi=dpi)
    return ax


def _fmt(v: float, precision: Optional[int]) -> str:
    return f"{v:.{precision}f}" if precision is not None and not isinstance(v, str) else str(v)


# ------------------------------------------------------------------ data ----
def importance_table(booster: Any, importance_type: str = "auto", max_num_features: Optional[int] = None, ignore_zero: bool = True) -> List[Tuple[str, float]]:
    """(feature name, importance) pairs, ascending (the order a horizontal bar chart draws them)."""
    est = booster
    bst = _booster_of(booster)
    if importance_type == "auto":
        importance_type = getattr(est, "importance_type", "split") if not isinstance(est, Booster) else "split"
    imp = bst.feature_importance(importance_type=importance_type)
    names = bst.feature_name()
    pairs = sorted(zip(names, imp), key=lambda p: p[1])
    if ignore_zero:
        pairs = [p for p in pairs if p[1] != 0]
    if max_num_features is not None and max_num_features > 0:
        pairs = pairs[-max_num_features:]
    if not pairs:
        raise ValueError("Booster's feature_importance is empty")
    return [(n, float(v)) for n, v in pairs]


def _walk(node: Dict[str, Any]):
    yield node
    for key in ("left_child", "right_child"):
        if key in node:
            yield from _walk(node[key])


def split_value_histogram(booster: Any, feature: Union[int, str], bins: Union[int, str, None] = None) -> Tuple[np.ndarray, np.ndarray]:
    """Histogram of the thresholds the model uses for one numerical feature: (counts, bin edges)."""
    bst = _booster_of(booster)
    model = bst.dump_model()
    names = model.get("feature_names", bst.feature_name())
    fidx = names.index(feature) if isinstance(feature, str) else int(feature)
    values: List[float] = []
    for t in model["tree_info"]:
        for nd in _walk(t["tree_structure"]):
            if "split_feature" in nd and nd["split_feature"] == fidx:
                if nd.get("decision_type") == "==":
                    raise ValueError("Cannot compute a split value histogram for a categorical feature")
                values.append(float(nd["threshold"]))
    if not values:
        raise ValueError(f"Feature {feature!r} was not used in splitting")
    if bins is None or (isinstance(bins, int) and bins <= 0):
        bins = min(len(set(values)), 64) or 1
    return np.histogram(np.asarray(values), bins=bins)


def metric_curves(evals: Any, metric: Optional[str] = None, dataset_names: Optional[List[str]] = None) -> Tuple[str, Dict[str, List[float]]]:
    """(metric name, {dataset name: values per iteration}) from a ``record_evaluation`` dict or a fitted estimator."""
    if hasattr(evals, "evals_result_"):
        evals = evals.evals_result_
    if not isinstance(evals, dict) or not evals:
        raise ValueError("eval results are empty: pass the dict filled by record_evaluation() or a fitted estimator")
    names = dataset_names or list(evals.keys())
    first = evals[names[0]]
    if metric is None:
        metric = next(iter(first.keys()))
    if metric not in first:
        raise KeyError(f"metric {metric!r} was not recorded")
    return metric, {n: list(evals[n][metric]) for n in names}


def tree_to_dot(booster: Any, tree_index: int = 0, show_info: Optional[List[str]] = None, precision: Optional[int] = 3, orientation: str = "horizontal",
                example_case: Any = None, max_category_values: int = 10) -> str:
    """DOT source of one tree. Internal nodes read ``name <= threshold`` (``name in {..}`` for categorical splits),
    leaves ``leaf k: value``; ``show_info`` adds split_gain / internal_value / internal_count / leaf_count ... lines;
    ``example_case`` (one row) highlights the path that row takes."""
    bst = _booster_of(booster)
    model = bst.dump_model()
    infos = model["tree_info"]
    if not 0 <= tree_index < len(infos):
        raise IndexError("tree_index is out of range")
    names = model.get("feature_names") or bst.feature_name()
    show = set(show_info or [])
    row = None
    if example_case is not None:
        row = np.asarray(example_case, dtype=np.float64).reshape(-1)
    lines = ["digraph Tree {", f'  graph [rankdir={"LR" if orientation == "horizontal" else "TB"}];', '  node [shape=rectangle, fontname="Helvetica"];']
    counter = [0]

    def goes_left(nd: Dict[str, Any]) -> bool:
        v = row[nd["split_feature"]]
        if nd.get("decision_type") == "==":
            cats = {int(c) for c in str(nd["threshold"]).split("||")}
            return (not np.isnan(v)) and int(v) in cats
        mt = nd.get("missing_type", "None")
        if (mt == "NaN" and np.isnan(v)) or (mt == "Zero" and (np.isnan(v) or abs(v) <= 1e-35)):
            return bool(nd.get("default_left", False))
        if np.isnan(v):
            v = 0.0
        return v <= float(nd["threshold"])

    def emit(nd: Dict[str, Any], on_path: bool) -> str:
        me = f"n{counter[0]}"; counter[0] += 1
        style = ', style=filled, fillcolor="lightblue"' if on_path else ""
        if "split_feature" in nd:
            fname = names[nd["split_feature"]] if nd["split_feature"] < len(names) else f"Column_{nd['split_feature']}"
            if nd.get("decision_type") == "==":
                cats = str(nd["threshold"]).split("||")
                shown = cats[:max_category_values] + (["..."] if len(cats) > max_category_values else [])
                label = f"{fname} in {{{', '.join(shown)}}}"
            else:
                label = f"{fname} <= {_fmt(float(nd['threshold']), precision)}"
            for key in ("split_gain", "internal_value", "internal_weight", "internal_count"):
                if key in show and key in nd:
                    label += f"\\n{key}: {_fmt(nd[key], precision) if isinstance(nd[key], float) else nd[key]}"
            lines.append(f'  {me} [label="{label}"{style}];')
            left_on = on_path and row is not None and goes_left(nd)
            right_on = on_path and row is not None and not goes_left(nd)
            l = emit(nd["left_child"], left_on); r = emit(nd["right_child"], right_on)
            lines.append(f'  {me} -> {l} [label="yes"];'); lines.append(f'  {me} -> {r} [label="no"];')
        else:
            label = f"leaf {nd.get('leaf_index', 0)}: {_fmt(float(nd['leaf_value']), precision)}"
            for key in ("leaf_weight", "leaf_count"):
                if key in show and key in nd:
                    label += f"\\n{key}: {_fmt(nd[key], precision) if isinstance(nd[key], float) else nd[key]}"
            lines.append(f'  {me} [label="{label}", shape=ellipse{style}];')
        return me

    emit(infos[tree_index]["tree_structure"], row is not None)
    lines.append("}")
    return "\n".join(lines)


# ----------------------------------------------------------------- plots ----
def plot_importance(booster: Any, ax: Any = None, height: float = 0.2, xlim: Optional[Tuple[float, float]] = None, ylim: Optional[Tuple[float, float]] = None,
                    title: Optional[str] = "Feature importance", xlabel: Optional[str] = "Feature importance", ylabel: Optional[str] = "Features",
                    importance_type: str = "auto", max_num_features: Optional[int] = None, ignore_zero: bool = True, figsize: Optional[Tuple[float, float]] = None,
                    dpi: Optional[int] = None, grid: bool = True, precision: Optional[int] = 3, **kwargs: Any) -> Any:
    pairs = importance_table(booster, importance_type, max_num_features, ignore_zero)
    labels, values = zip(*pairs)
    ax = _axes(ax, figsize, dpi)
    ylocs = np.arange(len(values))
    ax.barh(ylocs, values, align="center", height=height, **kwargs)
    for x, y in zip(values, ylocs):
        ax.text(x + 1, y, _fmt(x, precision) if importance_type == "gain" else str(int(x)) if float(x).is_integer() else _fmt(x, precision), va="center")
    ax.set_yticks(ylocs); ax.set_yticklabels(labels)
    ax.set_xlim(xlim if xlim is not None else (0, max(values) * 1.1)); ax.set_ylim(ylim if ylim is not None else (-1, len(values)))
    if title is not None: ax.set_title(title)
    if xlabel is not None: ax.set_xlabel(xlabel)
    if ylabel is not None: ax.set_ylabel(ylabel)
    ax.grid(grid)
    return ax


def plot_split_value_histogram(booster: Any, feature: Union[int, str], bins: Union[int, str, None] = None, ax: Any = None, width_coef: float = 0.8,
                               xlim: Optional[Tuple[float, float]] = None, ylim: Optional[Tuple[float, float]] = None,
                               title: Optional[str] = "Split value histogram for feature with @index/name@ @feature@", xlabel: Optional[str] = "Feature split value",
                               ylabel: Optional[str] = "Count", figsize: Optional[Tuple[float, float]] = None, dpi: Optional[int] = None, grid: bool = True,
                               **kwargs: Any) -> Any:
    hist, edges = split_value_histogram(booster, feature, bins)
    ax = _axes(ax, figsize, dpi)
    width = width_coef * (edges[1] - edges[0])
    centres = (edges[:-1] + edges[1:]) / 2
    ax.bar(centres, hist, align="center", width=width, **kwargs)
    if xlim is None:
        r = (edges[-1] - edges[0]) * 0.2
        xlim = (edges[0] - r, edges[-1] + r)
    ax.set_xlim(xlim); ax.set_ylim(ylim if ylim is not None else (0, max(hist) * 1.1))
    if title is not None:
        ax.set_title(title.replace("@feature@", str(feature)).replace("@index/name@", "name" if isinstance(feature, str) else "index"))
    if xlabel is not None: ax.set_xlabel(xlabel)
    if ylabel is not None: ax.set_ylabel(ylabel)
    ax.grid(grid)
    return ax


def plot_metric(booster: Any, metric: Optional[str] = None, dataset_names: Optional[List[str]] = None, ax: Any = None, xlim: Optional[Tuple[float, float]] = None,
                ylim: Optional[Tuple[float, float]] = None, title: Optional[str] = "Metric during training", xlabel: Optional[str] = "Iterations",
                ylabel: Optional[str] = "@metric@", figsize: Optional[Tuple[float, float]] = None, dpi: Optional[int] = None, grid: bool = True) -> Any:
    if isinstance(booster, Booster):
        raise TypeError("booster must be a dict from record_evaluation() or a fitted estimator")
    name, curves = metric_curves(booster, metric, dataset_names)
    ax = _axes(ax, figsize, dpi)
    n = 0
    for ds, vals in curves.items():
        ax.plot(range(len(vals)), vals, label=ds); n = max(n, len(vals))
    ax.legend(loc="best")
    ax.set_xlim(xlim if xlim is not None else (0, n))
    if ylim is not None: ax.set_ylim(ylim)
    if title is not None: ax.set_title(title)
    if xlabel is not None: ax.set_xlabel(xlabel)
    if ylabel is not None: ax.set_ylabel(ylabel.replace("@metric@", name))
    ax.grid(grid)
    return ax


def create_tree_digraph(booster: Any, tree_index: int = 0, show_info: Optional[List[str]] = None, precision: Optional[int] = 3, orientation: str = "horizontal",
                        example_case: Any = None, max_category_values: int = 10, **kwargs: Any) -> Any:
    """graphviz.Source of one tree (needs the graphviz package; :func:`tree_to_dot` gives the DOT text without it)."""
    try:
        import graphviz
    except ImportError as e:  # pragma: no cover - optional dependency
        raise ImportError("graphviz is needed for create_tree_digraph; tree_to_dot() returns the DOT source without it") from e
    return graphviz.Source(tree_to_dot(booster, tree_index, show_info, precision, orientation, example_case, max_category_values), **kwargs)


def plot_tree(booster: Any, ax: Any = None, tree_index: int = 0, figsize: Optional[Tuple[float, float]] = None, dpi: Optional[int] = None,
              show_info: Optional[List[str]] = None, precision: Optional[int] = 3, orientation: str = "horizontal", example_case: Any = None, **kwargs: Any) -> Any:
    import io

    ax = _axes(ax, figsize, dpi)
    graph = create_tree_digraph(booster, tree_index, show_info, precision, orientation, example_case, **kwargs)
    import matplotlib.image as mpimg

    ax.imshow(mpimg.imread(io.BytesIO(graph.pipe(format="png"))))
    ax.axis("off")
    return ax
