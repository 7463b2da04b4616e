"""Loads the in-tree native module, building it on first use.

``C`` is ``flexkv_b200._C``. On a machine with a GPU the module must load:
there is no Python fallback for any kernel, and a missing extension raises
instead of degrading silently.
"""
from __future__ import annotations

import importlib
import os


def _load():
    try:
        return importlib.import_module("flexkv_b200._C")
    except ImportError:
        if os.environ.get("FLEXKV_NO_AUTOBUILD") == "1":
            raise
        from . import _build
        _build.build(verbose=True)
        importlib.invalidate_caches()
        return importlib.import_module("flexkv_b200._C")


C = _load()
