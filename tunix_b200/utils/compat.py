"""Small compatibility helpers (tunix/utils/compat.py:40-92)."""
from __future__ import annotations

import functools
import warnings

import torch.nn as nn

ModuleList = nn.ModuleList


def alias_init_param(old_name: str, new_name: str):
    """Class decorator: accept the deprecated keyword `old_name` for `new_name` in `__init__`."""
    def deco(cls):
        orig = cls.__init__

        @functools.wraps(orig)
        def init(self, *a, **kw):
            if old_name in kw:
                if new_name in kw:
                    raise TypeError(f"pass {new_name!r} or its deprecated alias {old_name!r}, not both")
                warnings.warn(f"{cls.__name__}: {old_name!r} is deprecated, use {new_name!r}", DeprecationWarning, stacklevel=2)
                kw[new_name] = kw.pop(old_name)
            orig(self, *a, **kw)
        cls.__init__ = init
        return cls
    return deco


def set_mesh(mesh):
    from ..parallel import mesh as mesh_lib
    mesh_lib.set_mesh(mesh)
    return mesh
