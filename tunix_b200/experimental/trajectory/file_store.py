"""Step-level store on a file system (tunix/experimental/trajectory/file_store.py:110-673).

    <root>/<trajectory id>/metadata.json          ATIF metadata
    <root>/<trajectory id>/step_<000001>.json     one ATIF step per file

Writes are queued to a writer thread (`async_writer.AsyncWriter`); every file is written to a temporary name and
renamed, so a reader sees a step completely or not at all. Readers list the directories; a trajectory directory
without a metadata file (its first write is still queued) is not listed."""
from __future__ import annotations

import collections
import json
import os
import tempfile
import urllib.parse
from typing import List, Optional

from . import trajectory as T
from .async_writer import AsyncWriter
from .base_store import TrajectoryMetadataNotFoundError, TrajectoryNotFoundError, TrajectoryStore


def _safe(trajectory_id: str) -> str:
    """A directory name for any id (path separators and dots are escaped; the mapping is reversible)."""
    return urllib.parse.quote(trajectory_id, safe="") .replace(".", "%2E")


def _unsafe(name: str) -> str:
    return urllib.parse.unquote(name)


def _write_atomic(path: str, doc: dict) -> None:
    d = os.path.dirname(path)
    os.makedirs(d, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=d, prefix=".tmp_", suffix=".json")
    try:
        with os.fdopen(fd, "w") as f:
            json.dump(doc, f)
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


class _FileWriter(AsyncWriter):
    """Metadata that has not changed since it was last written for a trajectory is not written again (every `add_step`
    carries the metadata; during an episode it is mostly the same document)."""

    def __init__(self, name: str, max_queue_size: int):
        self._last_meta: "collections.OrderedDict[str, str]" = collections.OrderedDict()
        super().__init__(name, max_queue_size)

    def _process_task(self, task) -> None:
        for path, doc in task:
            if path.endswith("metadata.json"):
                text = json.dumps(doc, sort_keys=True)
                if self._last_meta.get(path) == text and os.path.isfile(path):
                    continue
                self._last_meta[path] = text
                self._last_meta.move_to_end(path)
                while len(self._last_meta) > 8192:
                    self._last_meta.popitem(last=False)
            _write_atomic(path, doc)


class FileTrajectoryStore(TrajectoryStore):
    STORE_TYPE = "file"

    def __init__(self, root_dir: str, max_queue_size: int = 4096):
        self._root = os.path.abspath(os.fspath(root_dir))
        os.makedirs(self._root, exist_ok=True)
        self._max_queue = max_queue_size
        self._writer: Optional[_FileWriter] = None
        self._closed = False

    def to_config(self) -> dict:
        return {"store_type": self.STORE_TYPE, "root_dir": self._root, "max_queue_size": self._max_queue}

    @property
    def root_dir(self) -> str:
        return self._root

    def get_trajectory_dir(self, trajectory_id: str) -> str:
        return os.path.join(self._root, _safe(trajectory_id))

    def get_trajectory_metadata_path(self, trajectory_id: str) -> str:
        return os.path.join(self.get_trajectory_dir(trajectory_id), "metadata.json")

    def get_step_path(self, trajectory_id: str, step_id: int) -> str:
        return os.path.join(self.get_trajectory_dir(trajectory_id), f"step_{step_id:06d}.json")

    # ---------------------------------------------------------------- reads
    def _list_ids(self) -> list:
        out = []
        for name in sorted(os.listdir(self._root)):
            if os.path.isfile(os.path.join(self._root, name, "metadata.json")):
                out.append(_unsafe(name))
        return out

    def _read(self, path: str) -> dict:
        with open(path) as f:
            return json.load(f)

    def get_trajectories_metadata(self, trajectory_ids: Optional[List[str]] = None) -> list:
        ids = self._list_ids() if trajectory_ids is None else list(trajectory_ids)
        out = []
        for t in ids:
            path = self.get_trajectory_metadata_path(t)
            if not os.path.isfile(path):
                raise TrajectoryMetadataNotFoundError(t)
            out.append(self._rehydrate_metadata(self._read(path)))
        return out

    def get_trajectories(self, trajectory_ids: List[str]) -> list:
        out = []
        for t in trajectory_ids:
            d, meta = self.get_trajectory_dir(t), self.get_trajectory_metadata_path(t)
            if not os.path.isfile(meta):
                raise TrajectoryNotFoundError(t)
            steps = [self._read(os.path.join(d, n)) for n in sorted(os.listdir(d)) if n.startswith("step_") and n.endswith(".json")]
            out.append(self._rehydrate_trajectory(self._read(meta), steps))
        return out

    # ---------------------------------------------------------------- writes
    def _w(self) -> _FileWriter:
        if self._closed:
            raise RuntimeError("the store is closed")
        if self._writer is None:
            self._writer = _FileWriter("trajectory-file-writer", self._max_queue)
        return self._writer

    def add_step(self, step: T.Step, metadata: T.TrajectoryMetadata) -> None:
        tid = self._check(metadata)
        sdoc, mdoc = self._step_doc(step), self._metadata_doc(metadata)
        # the step first: once the metadata file exists the trajectory is listed, and it should then have its step
        self._w()._enqueue([(self.get_step_path(tid, sdoc["step_id"]), sdoc), (self.get_trajectory_metadata_path(tid), mdoc)])

    def update_metadata(self, metadata: T.TrajectoryMetadata) -> None:
        tid = self._check(metadata)
        self._w()._enqueue([(self.get_trajectory_metadata_path(tid), self._metadata_doc(metadata))])

    def flush(self) -> None:
        if self._writer is not None:
            self._writer.flush()

    def close(self) -> None:
        self._closed = True
        if self._writer is not None:
            self._writer.close()
            self._writer = None

    @property
    def write_errors(self) -> int:
        return self._writer.errors if self._writer is not None else 0
