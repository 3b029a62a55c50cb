"""A pool of interchangeable workers with sticky routing
(`RoutingActorPool`, tunix/experimental/worker/remote_execution.py:1589-1700).

A request that carries a `route_key` (a conversation id, a prompt group) always goes to the same worker while the
set of workers is unchanged, so that the worker's prefix cache keeps hitting; requests without a key go round robin
to the least loaded worker. The key is placed with rendezvous (highest-random-weight) hashing over a
process-independent digest: when a worker leaves, only the keys it owned move; Python's own `hash()` is salted per
process and would scatter the keys after every restart. Workers that fail are taken out of rotation and the request
is retried on the next choice for its key."""
from __future__ import annotations

import hashlib
import threading
from typing import Any, Callable, Optional, Sequence


def stable_route_hash(key: Any, salt: str = "") -> int:
    """64-bit digest of `key` that is the same in every process and on every host."""
    return int.from_bytes(hashlib.blake2b(f"{salt}\x1f{key}".encode(), digest_size=8).digest(), "big")


class NoWorkerAvailable(RuntimeError):
    pass


class RoutingPool:
    def __init__(self, workers: Optional[dict] = None, *, call: Optional[Callable[[Any, Any], Any]] = None,
                 router: Optional[Callable[[Any, Sequence[str]], Optional[str]]] = None, max_attempts: int = 3):
        """`workers`: name -> worker. `call(worker, request)` performs one request (default: `worker.submit(request)`).
        `router(request, live_names)` may pick a worker by name itself; None falls through to key / round robin."""
        self._workers: dict = dict(workers or {})
        self._call = call or (lambda w, req: w.submit(req))
        self._router = router
        self._max_attempts = max_attempts
        self._lock = threading.Lock()
        self._inflight = {n: 0 for n in self._workers}
        self._served = {n: 0 for n in self._workers}
        self._down: set = set()
        self._rr = 0

    # ------------------------------------------------------------------ membership
    def add_worker(self, name: str, worker) -> None:
        with self._lock:
            self._workers[name] = worker
            self._inflight.setdefault(name, 0)
            self._served.setdefault(name, 0)
            self._down.discard(name)

    def remove_worker(self, name: str) -> None:
        with self._lock:
            self._workers.pop(name, None)
            self._down.discard(name)

    def mark_down(self, name: str) -> None:
        with self._lock:
            if name in self._workers:
                self._down.add(name)

    def mark_up(self, name: str) -> None:
        with self._lock:
            self._down.discard(name)

    def live(self) -> list:
        with self._lock:
            return sorted(n for n in self._workers if n not in self._down)

    # ------------------------------------------------------------------ routing
    @staticmethod
    def route_key_of(request: Any) -> Optional[Any]:
        if isinstance(request, dict):
            return request.get("route_key")
        return getattr(request, "route_key", None)

    def _ranked(self, key: Any, names: Sequence[str]) -> list:
        return sorted(names, key=lambda n: stable_route_hash(key, n), reverse=True)

    def owner(self, route_key: Any) -> str:
        names = self.live()
        if not names:
            raise NoWorkerAvailable("no live worker")
        return self._ranked(route_key, names)[0]

    def _choices(self, request: Any) -> list:
        names = self.live()
        if not names:
            raise NoWorkerAvailable("no live worker")
        if self._router is not None:
            pick = self._router(request, names)
            if pick is not None:
                if pick not in names:
                    raise NoWorkerAvailable(f"router chose {pick!r}, which is not live")
                return [pick] + [n for n in names if n != pick]
        key = self.route_key_of(request)
        if key is not None:
            return self._ranked(key, names)
        with self._lock:
            self._rr += 1
            start = self._rr
            load = dict(self._inflight)
        rot = [names[(start + i) % len(names)] for i in range(len(names))]
        return sorted(rot, key=lambda n: load.get(n, 0))           # stable: ties keep the rotation order

    def submit(self, request: Any) -> Any:
        last: Optional[BaseException] = None
        tried = 0
        for name in self._choices(request):
            if tried >= self._max_attempts:
                break
            with self._lock:
                worker = self._workers.get(name)
                if worker is None or name in self._down:
                    continue
                self._inflight[name] += 1
            tried += 1
            try:
                out = self._call(worker, request)
                with self._lock:
                    self._served[name] += 1
                return out
            except Exception as e:                          # this worker is out until someone marks it up again
                last = e
                self.mark_down(name)
            finally:
                with self._lock:
                    self._inflight[name] -= 1
        raise NoWorkerAvailable(f"request failed on {tried} worker(s)") from last

    def follow(self, monitor, period_s: float = 1.0) -> "threading.Event":
        """Keep this pool's rotation in step with a `HealthMonitor`: workers it reports unhealthy (silent, failed,
        stuck in a transitional state) are marked down before a request has to fail on them, and marked up again
        once their reports are healthy. Returns the event that stops the follower thread."""
        stop = threading.Event()

        def loop():
            while not stop.wait(period_s):
                self.apply_health(monitor)
        threading.Thread(target=loop, name="routing-pool-health", daemon=True).start()
        return stop

    def apply_health(self, monitor) -> tuple:
        """One pass of `follow`; returns (marked down, marked up)."""
        bad = {u.worker_id for u in monitor.check()}
        good = set(monitor.healthy_workers())
        with self._lock:
            names = set(self._workers)
            down = sorted((bad & names) - self._down)
            up = sorted(good & names & self._down)
            self._down |= set(down)
            self._down -= set(up)
        return down, up

    def stats(self) -> dict:
        with self._lock:
            return {n: {"served": self._served.get(n, 0), "inflight": self._inflight.get(n, 0), "down": n in self._down}
                    for n in self._workers}
