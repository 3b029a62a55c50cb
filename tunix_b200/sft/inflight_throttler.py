"""Bound the number of training steps queued on the device (tunix/sft/inflight_throttler.py:21-67).

Each step registers a CUDA event (or any object with `synchronize()`); when more than
`max_inflight` are outstanding the oldest is waited for.
"""
from __future__ import annotations

import collections


class InflightThrottler:
    def __init__(self, max_inflight: int = 2):
        if max_inflight is not None and max_inflight < 0:
            raise ValueError("max_inflight must be >= 0")
        self._max = max_inflight
        self._q = collections.deque()

    def add_computation(self, handle) -> None:
        if self._max is None or handle is None:
            return
        self._q.append(handle)

    def wait_for_next(self) -> None:
        if self._max is None:
            return
        while len(self._q) > self._max:
            self._q.popleft().synchronize()

    def wait_for_all(self) -> None:
        while self._q:
            self._q.popleft().synchronize()
