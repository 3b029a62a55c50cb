"""Process-environment helpers (role of tunix/utils/env_utils.py:22-45 on a torch.distributed box)."""
from __future__ import annotations

import os


def setup_distributed_environment(master_addr: str = "127.0.0.1", master_port: int = 29500) -> None:
    """Defaults for a single-node launch: loopback rendezvous and one visible process per GPU."""
    os.environ.setdefault("MASTER_ADDR", master_addr)
    os.environ.setdefault("MASTER_PORT", str(master_port))
    os.environ.setdefault("NCCL_NVLS_ENABLE", os.environ.get("NCCL_NVLS_ENABLE", "1"))


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def world_size() -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


def is_distributed_launch() -> bool:
    return "RANK" in os.environ and world_size() > 1


def is_internal_env() -> bool:
    return False
