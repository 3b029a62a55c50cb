"""Record-level trajectory stores (tunix/experimental/trajectory/*): an append-only record of rollouts for inspection
and replay. (The typed, step-level ATIF stores are `in_memory_store`, `file_store` and `sql_store` beside this module;
`open_store` gives the explorer a record view of those too.) Records are plain dicts (`trajectory_id`, `group_id`, `policy_version`, `steps`, `reward`, free-form
`metadata`); the in-memory store indexes them, the file store appends JSON lines through a writer thread so that
producers never wait on the disk."""
from __future__ import annotations

import json
import os
import queue
import threading
import time
import uuid
from typing import Callable, Iterator, Optional


def new_record(steps: list, reward: float = 0.0, group_id: Optional[str] = None, policy_version: int = 0, **metadata) -> dict:
    return {"trajectory_id": uuid.uuid4().hex, "group_id": group_id, "policy_version": policy_version, "steps": steps,
            "reward": float(reward), "created_at": time.time(), "metadata": metadata}


class InMemoryTrajectoryStore:
    def __init__(self, capacity: Optional[int] = None):
        self._items: "dict[str, dict]" = {}
        self._order: list = []
        self.capacity = capacity
        self._lock = threading.Lock()

    def put(self, record: dict) -> str:
        with self._lock:
            tid = record["trajectory_id"]
            self._items[tid] = record
            self._order.append(tid)
            while self.capacity and len(self._order) > self.capacity:
                self._items.pop(self._order.pop(0), None)
        return tid

    def get(self, trajectory_id: str) -> dict:
        return self._items[trajectory_id]

    def query(self, predicate: Optional[Callable[[dict], bool]] = None, group_id: Optional[str] = None,
              min_policy_version: Optional[int] = None) -> Iterator[dict]:
        with self._lock:
            items = [self._items[t] for t in self._order]
        for r in items:
            if group_id is not None and r.get("group_id") != group_id:
                continue
            if min_policy_version is not None and r.get("policy_version", 0) < min_policy_version:
                continue
            if predicate is None or predicate(r):
                yield r

    def __len__(self) -> int:
        return len(self._order)


class FileTrajectoryStore:
    """JSON-lines file with a background writer; `close()` (or `flush()`) makes everything durable."""

    _STOP = object()

    def __init__(self, path: str, default=None):
        self.path = path
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self._q: "queue.Queue" = queue.Queue()
        self._default = default or _to_jsonable
        self._error: Optional[BaseException] = None
        self._t = threading.Thread(target=self._run, name="trajectory-writer", daemon=True)
        self._t.start()

    def _run(self) -> None:
        with open(self.path, "a", encoding="utf-8") as f:
            while True:
                item = self._q.get()
                try:
                    if item is self._STOP:
                        return
                    if isinstance(item, threading.Event):
                        f.flush()
                        os.fsync(f.fileno())
                        item.set()
                        continue
                    f.write(json.dumps(item, default=self._default) + "\n")
                except BaseException as e:          # surfaced on the next put / flush
                    self._error = e
                finally:
                    self._q.task_done()

    def put(self, record: dict) -> str:
        if self._error is not None:
            raise RuntimeError("trajectory writer failed") from self._error
        self._q.put(record)
        return record["trajectory_id"]

    def flush(self) -> None:
        ev = threading.Event()
        self._q.put(ev)
        ev.wait()
        if self._error is not None:
            raise RuntimeError("trajectory writer failed") from self._error

    def close(self) -> None:
        self.flush()
        self._q.put(self._STOP)
        self._t.join()

    def read(self) -> Iterator[dict]:
        with open(self.path, encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)


def _to_jsonable(o):
    try:
        import numpy as np
        if isinstance(o, np.ndarray):
            return o.tolist()
        if isinstance(o, np.generic):
            return o.item()
    except ImportError:
        pass
    if hasattr(o, "tolist"):
        return o.tolist()
    if hasattr(o, "__dict__"):
        return o.__dict__
    return str(o)


class SqliteTrajectoryStore:
    """SQL store (tunix/experimental/trajectory/: the SQL back end): one row per trajectory with the fields that
    queries filter on as indexed columns and the whole record as JSON. Safe to use from several threads (one
    connection, one lock); a path of ":memory:" keeps it in RAM."""

    _SCHEMA = ("CREATE TABLE IF NOT EXISTS trajectories (trajectory_id TEXT PRIMARY KEY, group_id TEXT, policy_version INTEGER,"
               " reward REAL, num_steps INTEGER, created_at REAL, record TEXT NOT NULL);"
               "CREATE INDEX IF NOT EXISTS idx_group ON trajectories (group_id);"
               "CREATE INDEX IF NOT EXISTS idx_version ON trajectories (policy_version);")

    def __init__(self, path: str, default=None):
        import sqlite3
        if path != ":memory:":
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.path = path
        self._default = default or _to_jsonable
        self._lock = threading.Lock()
        self._db = sqlite3.connect(path, check_same_thread=False)
        self._db.executescript(self._SCHEMA)
        self._db.commit()

    def put(self, record: dict) -> str:
        return self.put_many([record])[0]

    def put_many(self, records) -> list:
        rows = [(r["trajectory_id"], None if r.get("group_id") is None else str(r["group_id"]), int(r.get("policy_version", 0)),
                 float(r.get("reward", 0.0)), len(r.get("steps") or ()), float(r.get("created_at", time.time())),
                 json.dumps(r, default=self._default)) for r in records]
        with self._lock:
            self._db.executemany("INSERT OR REPLACE INTO trajectories VALUES (?, ?, ?, ?, ?, ?, ?)", rows)
            self._db.commit()
        return [r[0] for r in rows]

    def get(self, trajectory_id: str) -> dict:
        with self._lock:
            row = self._db.execute("SELECT record FROM trajectories WHERE trajectory_id = ?", (trajectory_id,)).fetchone()
        if row is None:
            raise KeyError(trajectory_id)
        return json.loads(row[0])

    def query(self, predicate: Optional[Callable[[dict], bool]] = None, group_id: Optional[str] = None,
              min_policy_version: Optional[int] = None, min_reward: Optional[float] = None,
              max_reward: Optional[float] = None, limit: Optional[int] = None, newest_first: bool = False) -> Iterator[dict]:
        where, args = [], []
        for clause, v in (("group_id = ?", None if group_id is None else str(group_id)), ("policy_version >= ?", min_policy_version),
                          ("reward >= ?", min_reward), ("reward <= ?", max_reward)):
            if v is not None:
                where.append(clause)
                args.append(v)
        sql = "SELECT record FROM trajectories" + (" WHERE " + " AND ".join(where) if where else "") + \
              " ORDER BY created_at " + ("DESC" if newest_first else "ASC") + ", rowid"
        if limit is not None and predicate is None:
            sql += f" LIMIT {int(limit)}"
        with self._lock:
            rows = self._db.execute(sql, args).fetchall()
        n = 0
        for (raw,) in rows:
            r = json.loads(raw)
            if predicate is None or predicate(r):
                yield r
                n += 1
                if limit is not None and n >= limit:
                    return

    def stats(self) -> dict:
        """Per policy version: count, mean / min / max reward, mean number of steps."""
        with self._lock:
            rows = self._db.execute("SELECT policy_version, COUNT(*), AVG(reward), MIN(reward), MAX(reward), AVG(num_steps)"
                                    " FROM trajectories GROUP BY policy_version ORDER BY policy_version").fetchall()
        return {int(v): {"count": int(c), "reward_mean": a, "reward_min": lo, "reward_max": hi, "steps_mean": s}
                for v, c, a, lo, hi, s in rows}

    def __len__(self) -> int:
        with self._lock:
            return int(self._db.execute("SELECT COUNT(*) FROM trajectories").fetchone()[0])

    def flush(self) -> None:
        with self._lock:
            self._db.commit()

    def close(self) -> None:
        with self._lock:
            self._db.commit()
            self._db.close()


def record_from_trajectory(traj, group_id=None, policy_version: int = 0, **metadata) -> dict:
    """Convert an agent `Trajectory` (rl/agentic/agents/agent_types.py) to a store record: per step the model's
    response, the parsed action, the observation, reward and the token-level arrays when they were kept."""
    steps = []
    for s in getattr(traj, "steps", ()):
        act = getattr(s, "action", None)
        step = {"model_response": getattr(s, "model_response", ""), "thought": getattr(s, "thought", ""),
                "action": getattr(act, "action", act), "observation": getattr(s, "observation", None),
                "reward": float(getattr(s, "reward", 0.0)), "done": bool(getattr(s, "done", False)),
                "mc_return": float(getattr(s, "mc_return", 0.0))}
        for k in ("assistant_tokens", "assistant_masks", "env_tokens", "env_masks", "logprobs"):
            v = getattr(s, k, None)
            if v is not None:
                step[k] = v
        steps.append(step)
    status = getattr(traj, "status", None)
    last = traj.steps[-1] if getattr(traj, "steps", None) else None
    if last is not None and getattr(last, "chat_completions", None):
        # the whole conversation as chat messages: what the last call saw plus its answer
        metadata.setdefault("conversation", list(last.chat_completions) + [{"role": "assistant", "content": last.model_response}])
    rec = new_record(steps, reward=float(getattr(traj, "reward", 0.0)), group_id=group_id, policy_version=policy_version,
                     status=getattr(status, "name", status), task=getattr(traj, "task", None), **metadata)
    return rec


def record_from_atif(traj) -> dict:
    """The record form of a stored ATIF trajectory (`trajectory.TunixTrajectory`), as the explorer shows it."""
    from . import trajectory as T
    steps, conversation = [], []
    for s in traj.steps:
        if isinstance(s, T.TunixAgentStep):
            calls = [{"name": c.function_name, "arguments": c.arguments} for c in (s.tool_calls or [])]
            steps.append({"model_response": s.message, "thought": s.reasoning_content or "", "action": calls or None,
                          "observation": None, "reward": 0.0, "done": False, "mc_return": float(s.mc_return or 0.0)})
            conversation.append({"role": "assistant", "content": s.message})
        else:
            if steps and steps[-1]["observation"] is None and s.step_id > 0:
                steps[-1].update(observation=s.message, reward=float(getattr(s, "reward", None) or 0.0),
                                 done=bool(getattr(s, "done", None) or False))
            if s.message:
                conversation.append({"role": "system" if T.Source(s.source) == T.Source.SYSTEM else "user", "content": s.message})
    versions = getattr(traj, "target_policy_versions", None) or [0]
    return {"trajectory_id": traj.trajectory_id, "group_id": getattr(traj, "prompt_id", None), "policy_version": int(min(versions)),
            "steps": steps, "reward": float(getattr(traj, "total_reward", None) or 0.0), "created_at": None,
            "metadata": {"status": getattr(traj, "status", None), "group_index": getattr(traj, "group_index", None),
                         "session_id": traj.session_id, "conversation": conversation}}


class AtifRecordView:
    """Read-only record view over a step-level ATIF store, for the explorer."""

    def __init__(self, store):
        self._store = store

    def read(self) -> Iterator[dict]:
        for meta in self._store.get_trajectories_metadata():
            yield record_from_atif(self._store.get_trajectories([meta.trajectory_id])[0])

    def put(self, record: dict) -> str:
        raise TypeError("an ATIF store is written step by step (`add_step`), not from records")

    def close(self) -> None:
        self._store.close()


def open_store(path: str):
    """Open a store by what the path is: a directory (or `atif:<directory>`) -> ATIF file store, `atif:<sqlite URL or
    .db path>` -> ATIF SQL store (both as read-only record views), `.db` / `.sqlite` -> record-level SQL store, anything
    else -> record-level JSON lines."""
    if path.startswith("atif:") or os.path.isdir(path):
        target = path[len("atif:"):] if path.startswith("atif:") else path
        if os.path.isdir(target):
            from .file_store import FileTrajectoryStore as _AtifFiles
            return AtifRecordView(_AtifFiles(target))
        from .sql_store import SqlTrajectoryStore
        return AtifRecordView(SqlTrajectoryStore(target))
    return SqliteTrajectoryStore(path) if path.endswith((".db", ".sqlite", ".sqlite3")) else FileTrajectoryStore(path)
