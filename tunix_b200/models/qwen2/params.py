"""Checkpoint loading for Qwen 2.5 (and the DeepSeek-R1 distillations on it) (tunix/models/qwen2/{model,params}.py): Hugging Face safetensors directories through the family's key map."""
from __future__ import annotations

from ..safetensors_loader import create_model_from_safe_tensors as _create, key_map_for
from .model import FAMILIES


def create_model_from_safe_tensors(path: str, config, device=None, dtype=None):
    if config.family not in FAMILIES:
        raise ValueError(f"this loader serves {FAMILIES}, got a {config.family!r} configuration")
    return _create(path, config, device=device, dtype=dtype)


def key_mapping(config) -> list:
    """(pattern, replacement) pairs from checkpoint tensor names to this framework's parameter names."""
    return key_map_for(config)
