"""falcata_b200 — a Blackwell-native gradient-boosted decision tree framework.

Public surface (parity: python-package/falcata/__init__.py:L11-15, L81-84): ``Dataset``, ``Booster``,
``train``, ``cv``, callbacks, sklearn-style estimators (``LGBM*`` / ``Falcata*`` names), model
importers and plotting helpers.
"""
from .basic import DataSequence as Sequence
from .basic import get_pickle_format, set_pickle_format
from .basic import (Booster, Dataset, FalcataDeprecationWarning, FalcataError, network_free, network_init, LightGBMError, cuda_available, register_logger, get_num_threads, set_num_threads, set_time_tag,
                    time_tag_report)
from .callback import EarlyStopException, early_stopping, log_evaluation, record_evaluation, reset_parameter
from .engine import CVBooster, cv, train
from .importers import from_catboost, from_xgboost
from . import tuner
from .oblique import ObliquePool
from .plotting import create_tree_digraph, plot_importance, plot_metric, plot_split_value_histogram, plot_tree

__version__ = "0.1.0"

__all__ = ["Sequence", "get_pickle_format", "set_pickle_format", "from_xgboost", "from_catboost", "ObliquePool", "plot_importance", "plot_metric", "plot_split_value_histogram", "plot_tree", "create_tree_digraph","Dataset", "Booster", "CVBooster", "train", "cv", "FalcataError", "FalcataDeprecationWarning", "network_init", "network_free", "LightGBMError", "register_logger", "cuda_available", "set_time_tag", "set_num_threads", "get_num_threads", "time_tag_report",
           "early_stopping", "log_evaluation", "record_evaluation", "reset_parameter", "EarlyStopException"]

try:  # sklearn-style estimators are optional (scikit-learn may be absent)
    from .sklearn import (FalcataClassifier, FalcataModel, FalcataRanker, FalcataRegressor, LGBMClassifier, LGBMModel, LGBMRanker,
                          LGBMRegressor)

    __all__ += ["LGBMModel", "LGBMClassifier", "LGBMRegressor", "LGBMRanker", "FalcataModel", "FalcataClassifier", "FalcataRegressor", "FalcataRanker"]
except ImportError:  # pragma: no cover
    pass
