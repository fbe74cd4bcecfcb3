"""Loads the C++ runtime module and re-exports the cache manager's classes.

The classes live in C++ (`csrc/runtime/cache_manager.hpp`): `CacheManager` owns
the page pools of every layer group, the block table of every request and the
state slots; `GroupConfig` describes a group (page size, window, number of
pages); `StepLayout` says where the arrays of a packed step lie in the staging
buffer.  The module is compiled at first import.
"""
from __future__ import annotations

import importlib.util
import threading

_lock = threading.Lock()
_module = None


def runtime():
    """The compiled `_lab_runtime` module (built on first call)."""
    global _module
    with _lock:
        if _module is None:
            from ..kernels.build import runtime_module_path

            path = runtime_module_path()
            spec = importlib.util.spec_from_file_location("_lab_runtime", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _module = mod
        return _module


def __getattr__(name):
    if name in ("CacheManager", "GroupConfig", "StepLayout", "CapacityError", "StateError",
                "Scheduler", "PlanEntry", "Finished", "FinishReason"):
        return getattr(runtime(), name)
    raise AttributeError(name)
