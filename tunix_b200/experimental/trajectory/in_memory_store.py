"""Step-level store in process memory (tunix/experimental/trajectory/in_memory_store.py:29-181): for tests and for a
single-process run that inspects its own trajectories."""
from __future__ import annotations

import threading
from typing import List, Optional

from . import trajectory as T
from .base_store import TrajectoryMetadataNotFoundError, TrajectoryNotFoundError, TrajectoryStore


class InMemoryTrajectoryStore(TrajectoryStore):
    STORE_TYPE = "in_memory"

    def __init__(self) -> None:
        self._meta: dict = {}
        self._steps: dict = {}
        self._lock = threading.Lock()

    def to_config(self) -> dict:
        return {"store_type": self.STORE_TYPE}

    def get_trajectories_metadata(self, trajectory_ids: Optional[List[str]] = None) -> list:
        with self._lock:
            ids = list(self._meta) if trajectory_ids is None else list(trajectory_ids)
            for t in ids:
                if t not in self._meta:
                    raise TrajectoryMetadataNotFoundError(t)
            docs = [self._meta[t] for t in ids]
        return [self._rehydrate_metadata(d) for d in docs]

    def get_trajectories(self, trajectory_ids: List[str]) -> list:
        out = []
        with self._lock:
            for t in trajectory_ids:
                if t not in self._meta:
                    raise TrajectoryNotFoundError(t)
                out.append((self._meta[t], list(self._steps.get(t, {}).values())))
        return [self._rehydrate_trajectory(m, s) for m, s in out]

    def add_step(self, step: T.Step, metadata: T.TrajectoryMetadata) -> None:
        tid = self._check(metadata)
        sdoc, mdoc = self._step_doc(step), self._metadata_doc(metadata)      # snapshots
        with self._lock:
            self._meta[tid] = mdoc
            self._steps.setdefault(tid, {})[sdoc["step_id"]] = sdoc

    def update_metadata(self, metadata: T.TrajectoryMetadata) -> None:
        tid = self._check(metadata)
        mdoc = self._metadata_doc(metadata)
        with self._lock:
            self._meta[tid] = mdoc
