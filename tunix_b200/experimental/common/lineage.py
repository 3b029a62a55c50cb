"""Provenance of trajectories, batches and policies (tunix/experimental/common/lineage.py:25-124): every artefact
carries a tracking id, the ids it was made from, and a list of timestamped events."""
from __future__ import annotations

import dataclasses
import time
from typing import Any, Optional, Sequence


@dataclasses.dataclass(kw_only=True)
class LineageEvent:
    component: str              # e.g. "engine.dispatch", "worker.rollout", "orchestrator.assembler"
    operation: str              # e.g. "generate", "pack", "fwd_bwd"
    timestamp_s: float = dataclasses.field(default_factory=time.time)
    attributes: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(kw_only=True)
class LineageContext:
    tracking_id: str
    parent_tracking_ids: list = dataclasses.field(default_factory=list)
    events: list = dataclasses.field(default_factory=list)

    def add_event(self, component: str, operation: str, attributes: Optional[dict] = None) -> LineageEvent:
        ev = LineageEvent(component=component, operation=operation, attributes=dict(attributes or {}))
        self.events.append(ev)
        return ev

    @classmethod
    def merge(cls, batch_id: str, contexts: Sequence[Optional["LineageContext"]], component: str, operation: str,
              attributes: Optional[dict] = None) -> "LineageContext":
        """The context of something assembled from several upstream artefacts (a batch from trajectories): the
        parents are the distinct upstream ids in first-seen order."""
        parents = list(dict.fromkeys(c.tracking_id for c in contexts if c is not None and c.tracking_id))
        out = cls(tracking_id=batch_id, parent_tracking_ids=parents)
        out.add_event(component, operation, attributes)
        return out


def map_in_chunks(fn, chunk_size: Optional[int], *arrays: Any):
    """Apply `fn` to row chunks of the arrays and concatenate the results (bounds peak memory of scoring passes;
    tunix/experimental/common/batch_utils.py:22-64)."""
    import numpy as np
    if not arrays:
        raise ValueError("at least one array is needed")
    n = arrays[0].shape[0]
    if any(getattr(a, "ndim", 0) < 1 or a.shape[0] != n for a in arrays):
        raise ValueError("arrays need a leading batch dimension of the same size")
    if chunk_size is not None and chunk_size <= 0:
        raise ValueError("chunk_size must be positive")
    if not chunk_size or chunk_size >= n:
        return np.asarray(fn(*arrays))
    return np.concatenate([np.asarray(fn(*(a[s:s + chunk_size] for a in arrays))) for s in range(0, n, chunk_size)], axis=0)
