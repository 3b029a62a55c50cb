"""Gemma 1 and 2 under its own name (tunix/models/gemma/{model,params,params_safetensors}.py). The architecture is `models.transformer.Transformer` configured by
`ModelConfig`; this module gives the family's class name and lists its presets, so that code written as
`from <package>.models.gemma import model as lib; lib.Gemma(lib.ModelConfig.<preset>())` keeps working."""
from __future__ import annotations

from ..config import ModelConfig
from ..transformer import Transformer

FAMILIES = ('gemma', 'gemma2')


def presets() -> list:
    """Names of the `ModelConfig` class methods that build a configuration of this family."""
    out = []
    for name in dir(ModelConfig):
        if name.startswith("_") or name in ("replace", "from_dict", "to_dict"):
            continue
        fn = getattr(ModelConfig, name)
        if not callable(fn) or not getattr(fn, "__self__", None) is ModelConfig:
            continue
        try:
            cfg = fn()
        except TypeError:
            continue
        if isinstance(cfg, ModelConfig) and cfg.family in FAMILIES:
            out.append(name)
    return sorted(out)


class Gemma(Transformer):
    def __init__(self, config: ModelConfig, device=None, seed: int = 0, init: bool = True):
        if config.family not in FAMILIES:
            raise ValueError(f"Gemma takes a configuration of family {FAMILIES}, got {config.family!r}")
        super().__init__(config, device=device)
        if init:
            self.init_weights(seed)
