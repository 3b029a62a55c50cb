"""Bring-up and tear-down of every registered worker (tunix/experimental/orchestrator/lifecycle.py:44-110).

`bring_up()` starts all workers side by side (a worker's `start()` is initialise -> capture / warm-up -> READY); if
any of them fails, the ones that did come up are stopped again and one `LifecycleError` names every failure, so a
run never continues on half a cluster. `shutdown()` stops everything best effort and reports what could not be
stopped."""
from __future__ import annotations

import concurrent.futures as cf
from typing import Sequence


class LifecycleError(RuntimeError):
    def __init__(self, phase: str, failures: Sequence[tuple]):
        self.phase, self.failures = phase, list(failures)
        super().__init__(f"{phase} failed on {len(self.failures)} worker(s): " +
                         "; ".join(f"{wid}: {err!r}" for wid, err in self.failures))


class LifecycleDriver:
    def __init__(self, registry, max_workers: int = 32):
        self.registry, self.max_workers = registry, max_workers

    def _each(self, ids: Sequence[str], fn) -> list:
        failures = []
        with cf.ThreadPoolExecutor(max_workers=max(1, min(self.max_workers, len(ids) or 1))) as pool:
            futs = {}
            for wid in ids:
                try:
                    futs[pool.submit(fn, self.registry.get(wid))] = wid
                except KeyError:                            # unregistered meanwhile: nothing to do
                    continue
            for f in cf.as_completed(futs):
                try:
                    f.result()
                except Exception as e:
                    failures.append((futs[f], e))
        return sorted(failures, key=lambda t: t[0])

    def bring_up(self) -> None:
        """Workers that are already serving (launched processes start themselves before they announce) are left
        alone; the others are started side by side."""
        from ..common.datatypes import WorkerState

        def start(w):
            if w.state not in (WorkerState.READY, WorkerState.BUSY):
                w.start()
        ids = self.registry.worker_ids()
        failures = self._each(ids, start)
        if failures:
            failed = {wid for wid, _ in failures}
            self._each([i for i in ids if i not in failed], lambda w: w.stop())
            raise LifecycleError("bring_up", failures)

    def shutdown(self) -> None:
        failures = self._each(self.registry.worker_ids(), lambda w: w.stop())
        if failures:
            raise LifecycleError("shutdown", failures)
