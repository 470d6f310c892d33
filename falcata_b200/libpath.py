"""Locate and load the native core. The library is built in-tree (``falcata_b200/lib``); if it is
missing it is built on first import. Parity: python-package/falcata/libpath.py."""
from __future__ import annotations

import ctypes
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfalcata_core.so"


def find_lib_path() -> Path:
    import os

    override = os.environ.get("FALCATA_LIB")   # e.g. the sanitizer build made by ``python -m falcata_b200.build --sanitize``
    if override:
        return Path(override)
    if not _LIB_PATH.exists():
        from .build import build

        build()
    return _LIB_PATH


def load_lib() -> ctypes.CDLL:
    return ctypes.CDLL(str(find_lib_path()), mode=ctypes.RTLD_GLOBAL)
