"""Process launcher and discovery for the worker stack (tunix/experimental/distributed/runtime/*, in miniature).

The controller serves a `Directory` (worker id -> endpoint, roles) over the same gRPC layer the workers use and
starts one process per worker:

    python -m tunix_b200.experimental.runtime.launcher --factory pkg.module:make_worker --worker-id rollout-0 \\
           --directory 127.0.0.1:4000 [--arg key=value ...]

The child builds its worker with `factory(worker_id=..., **args)`, serves it on a free loopback port, starts it
and announces itself to the directory; the controller waits for the announcements and hands out `RemoteWorker`
proxies (`Launcher.workers()`), which register in a `WorkerRegistry` like local workers. A child leaves when its
parent closes its stdin (so a dead controller does not leave workers behind) or when `stop` arrives over the wire."""
from __future__ import annotations

import argparse
import importlib
import subprocess
import sys
import threading
import time
from typing import Optional

from ..worker.remote_execution import RemoteWorker, serve_worker


class Directory:
    """Who serves what where. Served remotely; every method is a plain call."""

    def __init__(self):
        self._lock = threading.Lock()
        self._entries: dict = {}

    def announce(self, worker_id: str, address: str, roles) -> int:
        with self._lock:
            self._entries[worker_id] = {"address": address, "roles": tuple(roles), "since": time.time()}
            return len(self._entries)

    def withdraw(self, worker_id: str) -> None:
        with self._lock:
            self._entries.pop(worker_id, None)

    def entries(self) -> dict:
        with self._lock:
            return {k: dict(v) for k, v in self._entries.items()}


class Launcher:
    def __init__(self, token: Optional[str] = None):
        self.directory = Directory()
        self.token = token
        self._server = serve_worker(self.directory, "127.0.0.1:0", token)
        self._procs: dict = {}

    @property
    def address(self) -> str:
        return self._server.address

    def launch(self, factory: str, worker_id: str, **args) -> subprocess.Popen:
        """Start a worker process; `factory` is `package.module:callable`."""
        cmd = [sys.executable, "-m", "tunix_b200.experimental.runtime.launcher", "--factory", factory, "--worker-id", worker_id,
               "--directory", self.address]
        if self.token:
            cmd += ["--token", self.token]
        for k, v in args.items():
            cmd += ["--arg", f"{k}={v}"]
        p = subprocess.Popen(cmd, stdin=subprocess.PIPE)
        self._procs[worker_id] = p
        return p

    def wait_for(self, worker_ids, timeout: float = 60.0) -> dict:
        deadline = time.time() + timeout
        want = set(worker_ids)
        while time.time() < deadline:
            have = self.directory.entries()
            if want <= set(have):
                return have
            dead = [w for w in want - set(have) if self._procs.get(w) is not None and self._procs[w].poll() is not None]
            if dead:
                raise RuntimeError(f"worker process(es) {dead} exited before announcing themselves")
            time.sleep(0.05)
        raise TimeoutError(f"workers {sorted(want - set(self.directory.entries()))} did not come up in {timeout} s")

    def workers(self) -> dict:
        return {wid: RemoteWorker(e["address"], self.token) for wid, e in self.directory.entries().items()}

    def shutdown(self, timeout: float = 10.0) -> None:
        for wid, p in self._procs.items():
            if p.poll() is None and p.stdin:
                try:
                    p.stdin.close()                 # the child watches its stdin and leaves when it closes
                except OSError:
                    pass
        for wid, p in self._procs.items():
            try:
                p.wait(timeout)
            except subprocess.TimeoutExpired:
                p.kill()                            # this exact child, by handle
        self._procs.clear()
        self._server.stop()


def _parse_args(argv):
    ap = argparse.ArgumentParser()
    ap.add_argument("--factory", required=True)
    ap.add_argument("--worker-id", required=True)
    ap.add_argument("--directory", required=True)
    ap.add_argument("--token", default=None)
    ap.add_argument("--arg", action="append", default=[])
    ap.add_argument("--bind", default="127.0.0.1:0", help="address the worker serves on (0.0.0.0:PORT inside a pod)")
    ap.add_argument("--advertise", default=None, help="address announced to the directory (POD_IP:PORT inside a pod)")
    ap.add_argument("--stay", action="store_true", help="run until SIGTERM / SIGINT instead of until stdin closes "
                    "(a pod has no controlling parent holding a pipe)")
    return ap.parse_args(argv)


def _coerce(v: str):
    for cast in (int, float):
        try:
            return cast(v)
        except ValueError:
            pass
    return {"true": True, "false": False, "none": None}.get(v.lower(), v)


def main(argv=None) -> int:
    a = _parse_args(argv)
    mod, fn = a.factory.split(":")
    factory = getattr(importlib.import_module(mod), fn)
    worker = factory(worker_id=a.worker_id, **{k: _coerce(v) for k, v in (kv.split("=", 1) for kv in a.arg)})
    server = serve_worker(worker, a.bind, a.token)
    worker.start()
    directory = RemoteWorker(a.directory, a.token)
    directory.announce(a.worker_id, a.advertise or server.address, worker.info().roles)
    try:
        if a.stay:
            import signal
            done = threading.Event()
            for sig in (signal.SIGTERM, signal.SIGINT):
                signal.signal(sig, lambda *_: done.set())
            done.wait()
        else:
            sys.stdin.read()                        # returns when the controller closes the pipe or exits
    finally:
        try:
            directory.withdraw(a.worker_id)
        except Exception:
            pass
        try:
            worker.stop()
        except Exception:
            pass
        server.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
