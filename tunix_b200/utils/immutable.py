"""Classes whose instances freeze after `__init__` (tunix/utils/immutable.py:20-60)."""
from __future__ import annotations

import abc


class ImmutableMeta(abc.ABCMeta):
    def __call__(cls, *a, **kw):
        obj = super().__call__(*a, **kw)
        object.__setattr__(obj, "_frozen", True)
        return obj


class Immutable(metaclass=ImmutableMeta):
    def __setattr__(self, k, v):
        if getattr(self, "_frozen", False):
            raise AttributeError(f"{type(self).__name__} is immutable; cannot set {k!r}")
        object.__setattr__(self, k, v)

    def __delattr__(self, k):
        if getattr(self, "_frozen", False):
            raise AttributeError(f"{type(self).__name__} is immutable; cannot delete {k!r}")
        object.__delattr__(self, k)
