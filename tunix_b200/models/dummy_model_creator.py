"""Random-init models without checkpoints (tunix/models/dummy_model_creator.py:29-92): what the benchmarks use."""
from __future__ import annotations

import torch

from .config import ModelConfig, get_config
from .transformer import create_model


def create_dummy_model(config_or_name, device=None, dtype=torch.bfloat16, seed: int = 0, tp=None, weight_shard=None):
    """Build a randomly initialised Transformer for `config_or_name` (a preset name or a ModelConfig). `tp` /
    `weight_shard` are parallel contexts (`parallel.tp.TPContext`, `parallel.fsdp3.CommContext`): the model is
    created whole with the seed, so every rank starts from the same weights, then sliced for this rank."""
    cfg = get_config(config_or_name) if isinstance(config_or_name, str) else config_or_name
    assert isinstance(cfg, ModelConfig)
    model = create_model(cfg.replace(dtype=dtype), device=device, seed=seed)
    if tp is not None:
        from ..parallel import tp as tp_lib
        tp_lib.apply_tensor_parallel(model, tp)
    if weight_shard is not None:
        from ..parallel import fsdp3
        fsdp3.apply_weight_sharding(model, weight_shard)
    return model
