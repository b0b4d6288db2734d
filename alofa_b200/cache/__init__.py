"""Paged caches: the host-side manager and the device-side storage."""
from .manager import CacheManager, GroupSpec  # noqa: F401


def __getattr__(name):
    if name in ("CacheStorage", "LayerCache", "StateCache", "group_windows"):
        from . import storage

        return getattr(storage, name)
    raise AttributeError(name)
