"""Paged cache bookkeeping.  `CacheManager` is the C++ one (csrc/host/host.cpp through
native.py) unless the environment says Q6K_HOST=python, which selects the Python twin in
manager.py; both follow the same rules and the tests run both."""
import os

from .manager import CacheManager as PyCacheManager, GroupSpec, OutOfPages, OutOfSlots, PagePool, SlotPool
from .native import NativeCacheManager


def use_native_host() -> bool:
    return os.environ.get("Q6K_HOST", "native").lower() != "python"


CacheManager = NativeCacheManager if use_native_host() else PyCacheManager
