"""``import falcata`` compatibility name: the public API of :mod:`falcata_b200` under the package
name that users of the reference project import (python-package/falcata/__init__.py)."""
from falcata_b200 import *  # noqa: F401,F403
from falcata_b200 import __all__, __version__  # noqa: F401
