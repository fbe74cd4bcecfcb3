"""Cache manager: pages, block tables, state slots (C++, `csrc/runtime/cache_manager.hpp`)."""
from .manager import CacheManager, CapacityError, GroupConfig, StateError, StepLayout, runtime

__all__ = ["CacheManager", "CapacityError", "GroupConfig", "StateError", "StepLayout", "runtime"]
