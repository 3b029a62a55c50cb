"""Step-windowed profiler (tunix/sft/profiler.py:25-186) on torch.profiler + NVTX ranges.

Process 0 only, one active trace at a time globally. `maybe_activate(step)` /
`maybe_deactivate(step)` are called by the trainer each step.
"""
from __future__ import annotations

import threading
from typing import Optional

import torch

from ..common.configs import ProfilerOptions

_active_lock = threading.Lock()
_active_owner = None


class Profiler:
    def __init__(self, initial_step: int, max_step: Optional[int], profiler_options: Optional[ProfilerOptions]):
        self._opts = profiler_options
        self._do_not_profile = profiler_options is None or not profiler_options.log_dir
        try:
            import torch.distributed as dist
            if dist.is_initialized() and dist.get_rank() != 0:
                self._do_not_profile = True
        except Exception:  # pragma: no cover
            pass
        self._prof = None
        if self._do_not_profile:
            self._first = self._last = -1
            return
        self._first = initial_step + profiler_options.skip_first_n_steps
        self._last = self._first + profiler_options.profiler_steps
        if max_step is not None:
            self._last = min(self._last, max_step)

    @property
    def should_profile(self) -> bool:
        return not self._do_not_profile

    def maybe_activate(self, step: int) -> None:
        global _active_owner
        if self._do_not_profile or step != self._first:
            return
        with _active_lock:
            if _active_owner is not None:
                return
            _active_owner = self
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(
            activities=acts, on_trace_ready=torch.profiler.tensorboard_trace_handler(self._opts.log_dir))
        self._prof.start()

    def maybe_deactivate(self, step: int) -> None:
        global _active_owner
        if self._prof is None or step != self._last:
            return
        self._prof.stop()
        self._prof = None
        with _active_lock:
            if _active_owner is self:
                _active_owner = None
