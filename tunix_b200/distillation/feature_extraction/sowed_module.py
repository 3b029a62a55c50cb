"""Capture intermediate activations of a model ("sowing", tunix/distillation/feature_extraction/sowed_module.py).

`sow_intermediates(model, layer_filter)` is a context manager that records, for every sub-module whose dotted
name matches, the module's output (first element for tuple outputs) during the forwards run inside it."""
from __future__ import annotations

import contextlib
import re
from typing import Callable, Union

import torch.nn as nn


@contextlib.contextmanager
def sow_intermediates(model: nn.Module, layer_filter: Union[str, Callable[[str, nn.Module], bool]]):
    match = (lambda n, m: re.fullmatch(layer_filter, n) is not None) if isinstance(layer_filter, str) else layer_filter
    store: dict = {}
    handles = []
    for name, mod in model.named_modules():
        if name and match(name, mod):
            def hook(_m, _inp, out, _name=name):
                store.setdefault(_name, []).append(out[0] if isinstance(out, tuple) else out)
            handles.append(mod.register_forward_hook(hook))
    try:
        yield store
    finally:
        for h in handles:
            h.remove()


def pop_sowed_intermediates(store: dict) -> dict:
    out = {k: v[-1] for k, v in store.items() if v}
    store.clear()
    return out
