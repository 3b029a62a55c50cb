"""Per-role profiling windows counted in invocations (tunix/rl/profiler/profiler.py:41-258).

A role (actor, rollout, reference, ...) calls `maybe_start(role)` / `maybe_stop(role)` around its work; the
profiler records invocations `[skip_first, skip_first + num_invocations)` of that role with `torch.profiler`
(CPU + CUDA activities) and writes a Chrome trace per role. Stopping waits for the device work launched inside
the window (an event recorded at stop time) on a helper thread, so the caller is not blocked. Only one window
is active at a time in a process, as in the reference.
"""
from __future__ import annotations

import dataclasses
import os
import threading
from typing import Optional

import torch


@dataclasses.dataclass
class RLProfilerOptions:
    log_dir: str = "/tmp/tunix_b200_profile"
    roles: tuple = ("actor",)
    skip_first_n_invocations: int = 1
    num_invocations: int = 1
    with_stack: bool = False


class RLProfiler:
    _active_lock = threading.Lock()

    def __init__(self, options: Optional[RLProfilerOptions]):
        self.options = options
        self._counts: dict = {}
        self._prof = None
        self._role = None
        self._writers: list = []

    def enabled_for(self, role: str) -> bool:
        return self.options is not None and role in self.options.roles

    def maybe_start(self, role: str) -> bool:
        if not self.enabled_for(role):
            return False
        n = self._counts.get(role, 0)
        self._counts[role] = n + 1
        o = self.options
        if n != o.skip_first_n_invocations or self._prof is not None:
            return False
        if not RLProfiler._active_lock.acquire(blocking=False):
            return False
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, with_stack=o.with_stack)
        self._prof.__enter__()
        self._role, self._left = role, o.num_invocations
        return True

    def maybe_stop(self, role: str) -> bool:
        if self._prof is None or role != self._role:
            return False
        self._left -= 1
        if self._left > 0:
            return False
        prof, self._prof = self._prof, None
        ev = None
        if torch.cuda.is_available():
            ev = torch.cuda.Event()
            ev.record()

        def finish():
            try:
                if ev is not None:
                    ev.synchronize()
                prof.__exit__(None, None, None)
                os.makedirs(self.options.log_dir, exist_ok=True)
                prof.export_chrome_trace(os.path.join(self.options.log_dir, f"{role}_trace.json"))
            finally:
                RLProfiler._active_lock.release()
        t = threading.Thread(target=finish, name=f"rl-profiler-{role}", daemon=True)
        t.start()
        self._writers.append(t)
        return True

    def wait(self) -> None:
        for t in self._writers:
            t.join()
        self._writers = []
