"""The step-level trajectory store interface (tunix/experimental/trajectory/base_store.py:30-396).

Writers log one step at a time together with the trajectory's metadata (`add_step`) or only the metadata
(`update_metadata`); both snapshot their arguments at the call, so a caller may keep changing its objects. Readers ask
for metadata (all trajectories or some ids) or whole trajectories; a reader never sees a half-written step. What is
persisted is plain ATIF (extensions packed); reads give back the metadata class the documents were written with
(`TrajectoryMetadata.resolve_subclass`) and its trajectory class.

A store describes itself as a config dict (`to_config`) from which `TrajectoryStore.from_config` builds an equal
store in another process; `to_redacted_config` is the form that may be logged (credentials in URLs removed)."""
from __future__ import annotations

import abc
from typing import Any, Dict, List, Mapping, Optional, Protocol, runtime_checkable

from . import trajectory as T


class TrajectoryNotFoundError(KeyError):
    def __init__(self, trajectory_id: str) -> None:
        super().__init__(f"Trajectory not found: {trajectory_id}")
        self.trajectory_id = trajectory_id


class TrajectoryMetadataNotFoundError(KeyError):
    def __init__(self, trajectory_id: str) -> None:
        super().__init__(f"Trajectory metadata not found: {trajectory_id}")
        self.trajectory_id = trajectory_id


@runtime_checkable
class TrajectoryReader(Protocol):
    def get_trajectories_metadata(self, trajectory_ids: Optional[List[str]] = None) -> list: ...
    def get_trajectories(self, trajectory_ids: List[str]) -> list: ...


@runtime_checkable
class TrajectoryWriter(Protocol):
    def add_step(self, step: T.Step, metadata: T.TrajectoryMetadata) -> None: ...
    def update_metadata(self, metadata: T.TrajectoryMetadata) -> None: ...
    def flush(self) -> None: ...
    def close(self) -> None: ...


_STORE_TYPES: Dict[str, type] = {}


class TrajectoryStore(abc.ABC):
    STORE_TYPE: str = ""

    def __init_subclass__(cls, **kw) -> None:
        super().__init_subclass__(**kw)
        if cls.STORE_TYPE:
            _STORE_TYPES[cls.STORE_TYPE] = cls

    # ---------------------------------------------------------------- documents
    @staticmethod
    def _check(metadata: T.TrajectoryMetadata) -> str:
        if not isinstance(metadata, T.TrajectoryMetadata):
            raise TypeError(f"metadata must be a TrajectoryMetadata, got {type(metadata).__name__}")
        if not metadata.trajectory_id:
            raise ValueError("metadata.trajectory_id must be set")
        return metadata.trajectory_id

    @staticmethod
    def _metadata_doc(metadata: T.TrajectoryMetadata) -> dict:
        """Plain ATIF metadata JSON (a full trajectory is cut down to its metadata)."""
        return metadata.to_atif_json()

    @staticmethod
    def _step_doc(step: T.Step) -> dict:
        return step.to_atif_json()

    @staticmethod
    def _rehydrate_metadata(doc: Mapping[str, Any]) -> T.TrajectoryMetadata:
        base = T.TrajectoryMetadata.from_json(dict(doc))
        cls = T.TrajectoryMetadata.resolve_subclass(base)
        return base if cls is T.TrajectoryMetadata else cls.from_atif_metadata(base)

    @classmethod
    def _rehydrate_trajectory(cls, meta_doc: Mapping[str, Any], step_docs: List[Mapping[str, Any]]) -> T.Trajectory:
        meta = cls._rehydrate_metadata(meta_doc)
        steps = [T.Step.from_json(dict(d)) for d in sorted(step_docs, key=lambda d: d["step_id"])]
        return meta.create_trajectory(steps)

    # ---------------------------------------------------------------- interface
    @abc.abstractmethod
    def get_trajectories_metadata(self, trajectory_ids: Optional[List[str]] = None) -> list: ...

    @abc.abstractmethod
    def get_trajectories(self, trajectory_ids: List[str]) -> list: ...

    @abc.abstractmethod
    def add_step(self, step: T.Step, metadata: T.TrajectoryMetadata) -> None: ...

    @abc.abstractmethod
    def update_metadata(self, metadata: T.TrajectoryMetadata) -> None: ...

    def flush(self) -> None:
        pass

    def close(self) -> None:
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    # ---------------------------------------------------------------- config
    @abc.abstractmethod
    def to_config(self) -> dict: ...

    def to_redacted_config(self) -> dict:
        return self.to_config()

    @classmethod
    def _from_config(cls, config: Mapping[str, Any]):
        kw = {k: v for k, v in config.items() if k != "store_type"}
        return cls(**kw)

    @classmethod
    def from_config(cls, config: Optional[Mapping[str, Any]]):
        """The store a config describes; None for no config. Called on a concrete class, the config's type must match."""
        if not config:
            return None
        kind = config.get("store_type")
        target = _STORE_TYPES.get(kind)
        if target is None:
            raise ValueError(f"unknown trajectory store type {kind!r}; known: {sorted(_STORE_TYPES)}")
        if cls is not TrajectoryStore and not issubclass(target, cls):
            raise ValueError(f"config describes a {kind!r} store, not a {cls.__name__}")
        return target._from_config(config)
