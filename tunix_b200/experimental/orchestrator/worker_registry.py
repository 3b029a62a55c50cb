"""Registry of live workers by id and role (tunix/experimental/orchestrator/worker_registry.py:28-159). A worker
describes itself through `info()` (id + roles); registration keeps a snapshot of that and the live handle."""
from __future__ import annotations

import dataclasses
import threading
from typing import Any, Iterator


@dataclasses.dataclass(frozen=True)
class WorkerInfo:
    worker_id: str
    roles: tuple
    address: str = ""
    attributes: dict = dataclasses.field(default_factory=dict)


class WorkerGroup:
    """The workers of one role, in id order."""

    def __init__(self, role: str, members: list):
        self.role, self._members = role, list(members)

    def members(self) -> list:
        return list(self._members)

    def is_empty(self) -> bool:
        return not self._members

    def __len__(self) -> int:
        return len(self._members)

    def __iter__(self) -> Iterator[Any]:
        return iter(self._members)


class WorkerRegistry:
    def __init__(self):
        self._lock = threading.Lock()
        self._workers: dict = {}
        self._infos: dict = {}

    def register(self, worker, override: bool = False) -> WorkerInfo:
        info = worker.info()
        if not info.roles:
            raise ValueError(f"worker {info.worker_id!r} declares no roles")
        with self._lock:
            if info.worker_id in self._workers and not override:
                raise ValueError(f"duplicate worker_id: {info.worker_id!r}")
            self._workers[info.worker_id], self._infos[info.worker_id] = worker, info
        return info

    def unregister(self, worker_id: str) -> None:
        with self._lock:
            del self._workers[worker_id]
            del self._infos[worker_id]

    def get(self, worker_id: str):
        with self._lock:
            return self._workers[worker_id]

    def info(self, worker_id: str) -> WorkerInfo:
        with self._lock:
            return self._infos[worker_id]

    def group(self, role: str) -> WorkerGroup:
        with self._lock:
            ids = sorted(i for i, inf in self._infos.items() if role in inf.roles)
            return WorkerGroup(role, [self._workers[i] for i in ids])

    def roles(self) -> set:
        with self._lock:
            return {r for inf in self._infos.values() for r in inf.roles}

    def worker_ids(self) -> list:
        with self._lock:
            return sorted(self._workers)

    def infos(self) -> list:
        with self._lock:
            return [self._infos[i] for i in sorted(self._infos)]

    def __len__(self) -> int:
        with self._lock:
            return len(self._workers)

    def __contains__(self, worker_id: str) -> bool:
        with self._lock:
            return worker_id in self._workers
