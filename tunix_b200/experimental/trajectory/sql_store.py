"""Step-level store in a SQL database (tunix/experimental/trajectory/sql_store.py:1-779), on SQLite.

    trajectories(trajectory_id PRIMARY KEY, metadata TEXT, created_at, updated_at)
    steps(trajectory_id, step_id, step TEXT, PRIMARY KEY (trajectory_id, step_id))

A step and its trajectory's metadata are written in one transaction by a writer thread; re-writing a step id replaces
it. Queries that the file layout cannot answer without reading everything are answered by the database:
`count_steps`, `find_trajectory_ids(prompt_id=..., status=..., min_total_reward=...)` over the JSON of the metadata."""
from __future__ import annotations

import json
import time
from typing import List, Optional

from . import trajectory as T
from .async_writer import AsyncWriter
from .base_store import TrajectoryMetadataNotFoundError, TrajectoryNotFoundError, TrajectoryStore
from .db_engine import EngineConfig, acquire_engine, redact_url

_SCHEMA = """
CREATE TABLE IF NOT EXISTS trajectories (trajectory_id TEXT PRIMARY KEY, metadata TEXT NOT NULL, created_at REAL NOT NULL,
                                         updated_at REAL NOT NULL);
CREATE TABLE IF NOT EXISTS steps (trajectory_id TEXT NOT NULL, step_id INTEGER NOT NULL, step TEXT NOT NULL,
                                  PRIMARY KEY (trajectory_id, step_id));
"""


class _SqlWriter(AsyncWriter):
    def __init__(self, handle, max_queue_size: int):
        self._h = handle
        super().__init__("trajectory-sql-writer", max_queue_size, max_batch=256)

    def _process_task(self, task) -> None:
        self._process_batch([task])

    def _process_batch(self, tasks: list) -> None:
        """One transaction for all waiting rows; of several metadata versions of a trajectory only the last is written."""
        now = time.time()
        metas = {tid: mdoc for tid, mdoc, _ in tasks}
        with self._h.lock:
            db = self._h.engine
            try:
                db.executemany("INSERT INTO trajectories VALUES (?, ?, ?, ?) ON CONFLICT(trajectory_id) DO UPDATE SET "
                               "metadata = excluded.metadata, updated_at = excluded.updated_at",
                               [(tid, json.dumps(m), now, now) for tid, m in metas.items()])
                db.executemany("INSERT OR REPLACE INTO steps VALUES (?, ?, ?)",
                               [(tid, int(s["step_id"]), json.dumps(s)) for tid, _, s in tasks if s is not None])
                db.commit()
            except BaseException:
                db.rollback()
                raise


class SqlTrajectoryStore(TrajectoryStore):
    STORE_TYPE = "sql"

    def __init__(self, url: str, max_queue_size: int = 4096, busy_timeout_ms: int = 30_000):
        self._cfg = EngineConfig(url=url, busy_timeout_ms=busy_timeout_ms)
        self._max_queue = max_queue_size
        self._h = acquire_engine(self._cfg)
        with self._h.lock:
            self._h.engine.executescript(_SCHEMA)
            self._h.engine.commit()
        self._writer: Optional[_SqlWriter] = None
        self._closed = False

    def to_config(self) -> dict:
        return {"store_type": self.STORE_TYPE, "url": self._cfg.url, "max_queue_size": self._max_queue,
                "busy_timeout_ms": self._cfg.busy_timeout_ms}

    def to_redacted_config(self) -> dict:
        return {**self.to_config(), "url": redact_url(self._cfg.url)}

    # ---------------------------------------------------------------- reads
    def _q(self, sql: str, args=()) -> list:
        with self._h.lock:
            return self._h.engine.execute(sql, args).fetchall()

    def get_trajectories_metadata(self, trajectory_ids: Optional[List[str]] = None) -> list:
        if trajectory_ids is None:
            rows = self._q("SELECT metadata FROM trajectories ORDER BY created_at, trajectory_id")
            return [self._rehydrate_metadata(json.loads(r[0])) for r in rows]
        out = []
        for t in trajectory_ids:
            rows = self._q("SELECT metadata FROM trajectories WHERE trajectory_id = ?", (t,))
            if not rows:
                raise TrajectoryMetadataNotFoundError(t)
            out.append(self._rehydrate_metadata(json.loads(rows[0][0])))
        return out

    def get_trajectories(self, trajectory_ids: List[str]) -> list:
        out = []
        for t in trajectory_ids:
            rows = self._q("SELECT metadata FROM trajectories WHERE trajectory_id = ?", (t,))
            if not rows:
                raise TrajectoryNotFoundError(t)
            steps = [json.loads(r[0]) for r in self._q("SELECT step FROM steps WHERE trajectory_id = ? ORDER BY step_id", (t,))]
            out.append(self._rehydrate_trajectory(json.loads(rows[0][0]), steps))
        return out

    def count_steps(self, trajectory_id: str) -> int:
        return int(self._q("SELECT COUNT(*) FROM steps WHERE trajectory_id = ?", (trajectory_id,))[0][0])

    def find_trajectory_ids(self, *, prompt_id: Optional[str] = None, status: Optional[str] = None,
                            min_total_reward: Optional[float] = None, limit: Optional[int] = None) -> list:
        """Ids whose packed RL metadata match, oldest first."""
        ext = f"$.extra.{T.TUNIX_EXTENSIONS_KEY}"
        where, args = [], []
        for key, val, op in (("prompt_id", prompt_id, "="), ("status", status, "="), ("total_reward", min_total_reward, ">=")):
            if val is not None:
                where.append(f"json_extract(metadata, '{ext}.{key}') {op} ?")
                args.append(val)
        sql = "SELECT trajectory_id FROM trajectories" + (" WHERE " + " AND ".join(where) if where else "") + \
            " ORDER BY created_at, trajectory_id" + (f" LIMIT {int(limit)}" if limit else "")
        return [r[0] for r in self._q(sql, tuple(args))]

    # ---------------------------------------------------------------- writes
    def _w(self) -> _SqlWriter:
        if self._closed:
            raise RuntimeError("the store is closed")
        if self._writer is None:
            self._writer = _SqlWriter(self._h, self._max_queue)
        return self._writer

    def add_step(self, step: T.Step, metadata: T.TrajectoryMetadata) -> None:
        tid = self._check(metadata)
        self._w()._enqueue((tid, self._metadata_doc(metadata), self._step_doc(step)))

    def update_metadata(self, metadata: T.TrajectoryMetadata) -> None:
        tid = self._check(metadata)
        self._w()._enqueue((tid, self._metadata_doc(metadata), None))

    def flush(self) -> None:
        if self._writer is not None:
            self._writer.flush()

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        if self._writer is not None:
            self._writer.close()
            self._writer = None
        self._h.release()

    @property
    def write_errors(self) -> int:
        return self._writer.errors if self._writer is not None else 0
