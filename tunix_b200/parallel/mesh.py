"""Named device meshes over `torch.distributed` ranks.

The reference describes parallelism with a JAX `Mesh` whose named axes (`fsdp`, `tp`, optional `sp`;
`ep` aliased onto `fsdp`) appear in every tensor's PartitionSpec (tunix/utils/mesh.py:51,
tunix/models/llama3/model.py:47-82) and carves per-role sub-meshes out of the device pool
(`allocate_named_mesh_device_slices`, tunix/utils/mesh.py). On one NVSwitch box every GPU is
equidistant, so a mesh is simply an N-d array of ranks; each axis yields one process group per line.

    mesh = create_mesh((2, 4), ("fsdp", "tp"))       # all ranks call this
    mesh.group("tp"), mesh.axis_rank("tp"), mesh.axis_size("fsdp")
    slices = allocate_named_mesh_device_slices({"actor": 4, "rollout": 4})   # role -> rank list
"""
from __future__ import annotations

import ast
import math
from typing import Optional, Sequence

import numpy as np
import torch.distributed as dist

_CURRENT: Optional["Mesh"] = None


class Mesh:
    def __init__(self, shape: Sequence[int], axis_names: Sequence[str], ranks: Optional[Sequence[int]] = None):
        shape = tuple(int(s) for s in shape)
        if len(shape) != len(axis_names):
            raise ValueError(f"mesh shape {shape} and axis names {tuple(axis_names)} differ in length")
        n = int(np.prod(shape))
        ranks = list(range(n)) if ranks is None else list(ranks)
        if len(ranks) != n:
            raise ValueError(f"mesh of shape {shape} needs {n} ranks, got {len(ranks)}")
        self.shape, self.axis_names = shape, tuple(axis_names)
        self.devices = np.asarray(ranks, dtype=np.int64).reshape(shape)
        self._groups: dict = {}
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        if dist.is_initialized() and n > 1:
            self._build_groups()

    @property
    def size(self) -> int:
        return int(self.devices.size)

    @property
    def empty(self) -> bool:
        return self.size <= 1

    def contains(self, rank: Optional[int] = None) -> bool:
        rank = self.rank if rank is None else rank
        return bool((self.devices == rank).any())

    def coords(self, rank: Optional[int] = None) -> tuple:
        rank = self.rank if rank is None else rank
        idx = np.argwhere(self.devices == rank)
        if len(idx) == 0:
            raise ValueError(f"rank {rank} is not part of this mesh")
        return tuple(int(i) for i in idx[0])

    def _build_groups(self) -> None:
        # every rank must create every group, in the same order
        for ax, name in enumerate(self.axis_names):
            moved = np.moveaxis(self.devices, ax, -1).reshape(-1, self.shape[ax])
            for line in moved:
                members = [int(r) for r in line]
                g = dist.new_group(members) if len(members) > 1 else None
                if self.rank in members:
                    self._groups[name] = (g, members)
        members = [int(r) for r in self.devices.reshape(-1)]
        whole = None if members == list(range(self.world)) else dist.new_group(members)     # None = the default group
        if self.rank in members:
            self._groups["__all__"] = (whole, members)

    def axis_size(self, name: str) -> int:
        return self.shape[self.axis_names.index(name)] if name in self.axis_names else 1

    def axis_rank(self, name: str) -> int:
        if name not in self.axis_names or not self.contains():
            return 0
        return self.coords()[self.axis_names.index(name)]

    def group(self, name: str):
        return self._groups.get(name, (None, [self.rank]))[0]

    def all_group(self):
        """Process group of every rank of the mesh (None when that is the default group)."""
        return self._groups.get("__all__", (None, [self.rank]))[0]

    def group_ranks(self, name: str) -> list:
        return self._groups.get(name, (None, [self.rank]))[1]

    def data_parallel_rank_size(self, axes=("fsdp",)) -> tuple[int, int]:
        """Position and extent of this rank along the batch-sharding axes."""
        rank, size = 0, 1
        for a in axes:
            if a in self.axis_names:
                rank = rank * self.axis_size(a) + self.axis_rank(a)
                size *= self.axis_size(a)
        return rank, size

    def __enter__(self):
        global _CURRENT
        self._prev, _CURRENT = _CURRENT, self
        return self

    def __exit__(self, *exc):
        global _CURRENT
        _CURRENT = self._prev

    def __repr__(self):
        return f"Mesh(shape={self.shape}, axis_names={self.axis_names})"


def create_mesh(shape: Sequence[int] | str, axis_names: Sequence[str] | str, ranks: Optional[Sequence[int]] = None,
                set_current: bool = True) -> Mesh:
    """`shape` / `axis_names` may be tuples or their string forms ("(2,4)", "('fsdp','tp')") as in the CLI."""
    global _CURRENT
    if isinstance(shape, str):
        shape = ast.literal_eval(shape)
    if isinstance(axis_names, str):
        axis_names = ast.literal_eval(axis_names)
    if isinstance(shape, int):
        shape = (shape,)
    m = Mesh(shape, axis_names, ranks)
    if set_current:
        _CURRENT = m
    return m


def current_mesh() -> Optional[Mesh]:
    return _CURRENT


def set_mesh(mesh: Optional[Mesh]) -> None:
    global _CURRENT
    _CURRENT = mesh


def allocate_named_mesh_device_slices(requests: dict, num_devices: Optional[int] = None,
                                      allocation_policy: str = "COMPACT") -> dict:
    """Carve contiguous rank ranges for named roles out of the pool.

    requests: {name: count or mesh shape}. Names with identical requests may share devices when the pool is
    too small for disjoint slices only if the caller asks for it by giving the same name. Returns
    {name: [ranks]} (COMPACT: first-fit contiguous; PERFORMANCE: slices aligned to their own size, which
    keeps power-of-two groups on aligned rank boundaries).
    """
    if num_devices is None:
        num_devices = dist.get_world_size() if dist.is_initialized() else 1
    out, cursor = {}, 0
    for name, req in requests.items():
        n = int(np.prod(req)) if not isinstance(req, int) else int(req)
        if n <= 0:
            raise ValueError(f"role {name!r} requests {n} devices")
        if allocation_policy.upper() == "PERFORMANCE":
            cursor = int(math.ceil(cursor / n) * n)
        if cursor + n > num_devices:
            raise ValueError(f"cannot allocate {n} devices for {name!r}: {num_devices - cursor} of {num_devices} left")
        out[name] = list(range(cursor, cursor + n))
        cursor += n
    return out
