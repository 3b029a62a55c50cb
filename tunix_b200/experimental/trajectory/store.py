"""Trajectory stores (tunix/experimental/trajectory/*): an append-only record of rollouts for inspection and
replay. Records are plain dicts (`trajectory_id`, `group_id`, `policy_version`, `steps`, `reward`, free-form
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
