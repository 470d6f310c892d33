"""``import falcata`` compatibility name: the public API of :mod:`falcata_b200` under the package
name that users of the reference project import (python-package/falcata/__init__.py), submodules included
(``falcata.importers``, ``falcata.plotting``, ``falcata.sklearn`` ...)."""
import importlib as _importlib
import sys as _sys

from falcata_b200 import *  # noqa: F401,F403
from falcata_b200 import __all__, __version__  # noqa: F401

for _name in ("basic", "engine", "callback", "sklearn", "importers", "plotting", "oblique", "parallel", "ops", "utils", "tuner"):
    try:
        _module = _importlib.import_module(f"falcata_b200.{_name}")
        _sys.modules[f"{__name__}.{_name}"] = _module
        globals().setdefault(_name, _module)   # `falcata.<submodule>` works as an attribute too
    except ImportError:  # optional dependency of that submodule is absent
        pass
