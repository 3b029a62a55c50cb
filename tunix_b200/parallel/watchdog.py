"""Rank-health watchdog on the host: heartbeats through the `torch.distributed` store.

Every rank runs a small thread that writes `hb/<rank> = <monotonic counter>` every `interval_s`; any rank can ask
`dead_ranks()` for the peers whose counter has not moved for `timeout_s`. A training loop calls `check()` between
steps (never inside one): it raises `RankFailure` naming the silent ranks, so the survivors stop launching
kernels that would wait for a peer that is gone and fall back to checkpoint-and-exit. This is the host half of
failure detection; the device half is that every wait in the kernels is bounded and reports through the status
word (`_lib.raise_if_kernel_error`)."""
from __future__ import annotations

import threading
import time
from typing import Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    def __init__(self, ranks):
        super().__init__(f"ranks {sorted(ranks)} stopped sending heartbeats")
        self.ranks = sorted(ranks)


class Watchdog:
    def __init__(self, store=None, rank: Optional[int] = None, world: Optional[int] = None, interval_s: float = 1.0,
                 timeout_s: float = 10.0, prefix: str = "hb"):
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.interval_s, self.timeout_s, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._seen: dict = {}
        self._thread: Optional[threading.Thread] = None
        self._beat = 0

    def start(self) -> "Watchdog":
        self._write()
        self._thread = threading.Thread(target=self._run, name=f"watchdog-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def _write(self) -> None:
        self._beat += 1
        self.store.set(f"{self.prefix}/{self.rank}", str(self._beat))

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            if not self._paused.is_set():
                try:
                    self._write()
                except Exception:
                    return

    def pause(self) -> None:
        """Stop beating without stopping the thread (tests use it to play a hung rank)."""
        self._paused.set()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)

    def dead_ranks(self) -> list:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            key = f"{self.prefix}/{r}"
            try:
                val = self.store.get(key).decode() if self.store.check([key]) else None
            except Exception:
                val = None
            last = self._seen.get(r)
            if last is None or last[0] != val:
                self._seen[r] = (val, now)
            elif now - last[1] > self.timeout_s:
                dead.append(r)
        return dead

    def check(self) -> None:
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead)
