"""Batch sharding across data-parallel ranks (tunix/sft/sharding_utils.py:25-97).

The reference builds global arrays from host-local data along `data_sharding_axis`. With one
process per GPU the analogue is: every rank receives the same global batch from its iterator and
keeps rows [rank * B/N, (rank+1) * B/N) of every array whose leading dim is divisible by the
data-parallel size; other leaves are replicated (same fallback rule as the reference).
"""
from __future__ import annotations

import dataclasses
from typing import Any

import numpy as np
import torch


def _dp_info(axes, model_parallel: int = 1) -> tuple[int, int]:
    try:
        from ..parallel import mesh as mesh_lib
        m = mesh_lib.current_mesh()
        if m is not None:
            return m.data_parallel_rank_size(axes)
    except Exception:
        pass
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            # without a mesh, ranks of one model-parallel (tensor-parallel) group are adjacent and share a batch
            return dist.get_rank() // model_parallel, dist.get_world_size() // model_parallel
    except Exception:
        pass
    return 0, 1


def _shard_leaf(x, rank: int, size: int):
    if isinstance(x, (np.ndarray, torch.Tensor)) and x.ndim >= 1 and x.shape[0] % size == 0 and x.shape[0] >= size:
        n = x.shape[0] // size
        return x[rank * n:(rank + 1) * n]
    return x


def shard_input(batch: Any, data_sharding_axis=("fsdp",), already_local: bool = False, model_parallel: int = 1) -> Any:
    rank, size = _dp_info(data_sharding_axis, model_parallel)
    if size == 1 or already_local or getattr(batch, "_is_local_shard", False):
        return batch
    if isinstance(batch, dict):
        if batch.get("_is_local_shard"):
            return batch
        return {k: _shard_leaf(v, rank, size) for k, v in batch.items()}
    if dataclasses.is_dataclass(batch) and not isinstance(batch, type):
        return dataclasses.replace(batch, **{f.name: _shard_leaf(getattr(batch, f.name), rank, size)
                                             for f in dataclasses.fields(batch)})
    return _shard_leaf(batch, rank, size)
