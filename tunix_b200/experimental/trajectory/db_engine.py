"""Database handles for the SQL trajectory store (tunix/experimental/trajectory/db_engine.py:12-204). Only SQLite is
built in (the standard library's driver): `sqlite:///relative.db`, `sqlite:////absolute.db`, `sqlite://` or
`sqlite:///:memory:` for a private in-memory database, or a bare file path. Handles to the same file are shared and
reference counted inside a process; file databases run in WAL mode with a busy timeout, so that a reader in another
process does not block the writer."""
from __future__ import annotations

import dataclasses
import enum
import os
import re
import sqlite3
import threading
from typing import Callable, Dict, Tuple


class Dialect(str, enum.Enum):
    SQLITE = "sqlite"


@dataclasses.dataclass(frozen=True)
class EngineConfig:
    url: str
    busy_timeout_ms: int = 30_000
    synchronous: str = "NORMAL"

    def path(self) -> str:
        """The file path (":memory:" for in-memory databases)."""
        u = self.url
        if "://" not in u:
            return u
        scheme, rest = u.split("://", 1)
        if scheme.split("+")[0] != Dialect.SQLITE.value:
            raise ValueError(f"unsupported database dialect in {redact_url(u)!r}: only sqlite is built in")
        if rest in ("", "/:memory:"):
            return ":memory:"
        if not rest.startswith("/"):
            raise ValueError(f"malformed sqlite URL {u!r}: use sqlite:///relative/path or sqlite:////absolute/path")
        return rest[1:]

    @property
    def in_memory(self) -> bool:
        return self.path() == ":memory:"


def redact_url(url: str) -> str:
    """The URL with the password of `scheme://user:password@host/...` replaced by `***`."""
    return re.sub(r"(://[^:/@]+):[^@/]+@", r"\1:***@", url)


def create_trajectory_engine(config: EngineConfig) -> sqlite3.Connection:
    path = config.path()
    if path != ":memory:":
        os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    db = sqlite3.connect(path, check_same_thread=False, timeout=config.busy_timeout_ms / 1000.0)
    db.execute(f"PRAGMA busy_timeout={int(config.busy_timeout_ms)}")
    db.execute("PRAGMA foreign_keys=ON")
    if path != ":memory:":
        db.execute("PRAGMA journal_mode=WAL")
        db.execute(f"PRAGMA synchronous={config.synchronous}")
    return db


_shared: Dict[str, Tuple[sqlite3.Connection, int, threading.RLock]] = {}
_shared_lock = threading.Lock()


class EngineHandle:
    """A connection plus the lock that serialises its use, released exactly once."""

    def __init__(self, engine: sqlite3.Connection, lock: threading.RLock, release_fn: Callable[[], None]):
        self._engine, self.lock, self._release, self._released = engine, lock, release_fn, False

    @property
    def engine(self) -> sqlite3.Connection:
        if self._released:
            raise RuntimeError("the engine handle has been released")
        return self._engine

    def release(self) -> None:
        if not self._released:
            self._released = True
            self._release()


def acquire_engine(config: EngineConfig) -> EngineHandle:
    if config.in_memory:                                        # private: every store gets its own database
        db = create_trajectory_engine(config)
        return EngineHandle(db, threading.RLock(), db.close)
    key = os.path.abspath(config.path())
    with _shared_lock:
        if key in _shared:
            db, n, lock = _shared[key]
            _shared[key] = (db, n + 1, lock)
        else:
            db, lock = create_trajectory_engine(config), threading.RLock()
            _shared[key] = (db, 1, lock)

    def release() -> None:
        with _shared_lock:
            db_, n_, lock_ = _shared[key]
            if n_ <= 1:
                del _shared[key]
                with lock_:
                    db_.commit()
                    db_.close()
            else:
                _shared[key] = (db_, n_ - 1, lock_)
    return EngineHandle(db, lock, release)
