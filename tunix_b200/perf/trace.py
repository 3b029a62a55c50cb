"""Always-on span tracer (tunix/perf/trace.py:114-471, tunix/perf/experimental/tracer.py).

    tracer = PerfTracer()
    with tracer.span_group("global_step"):
        with tracer.span("rollout", device=True):
            ...
Host spans measure wall clock. Device spans record a CUDA event on the current stream at entry and exit, so
their duration is time on the GPU ("timed on the device"), resolved lazily: no watcher thread and no
synchronisation in the hot loop (the reference blocks a thread on `block_until_ready`, :364-411).
Spans carry free-form tags (step / mini / micro / role), are grouped per thread ("timeline") and can be
exported as a Chrome/Perfetto trace (`perf/perfetto.py`) or reduced to metrics (`perf/export.py`).
"""
from __future__ import annotations

import contextlib
import dataclasses
import threading
import time
from typing import Any, Optional

import torch


@dataclasses.dataclass
class Span:
    name: str
    begin: float                       # host perf_counter seconds
    end: Optional[float] = None
    tags: dict = dataclasses.field(default_factory=dict)
    parent: Optional["Span"] = None
    timeline: str = "host"
    ev_begin: Any = None
    ev_end: Any = None
    _device_ms: Optional[float] = None

    @property
    def duration(self) -> float:
        return (self.end if self.end is not None else time.perf_counter()) - self.begin

    @property
    def device_duration(self) -> Optional[float]:
        """Seconds on the GPU between the two recorded events (None for host-only spans)."""
        if self.ev_begin is None or self.ev_end is None:
            return None
        if self._device_ms is None:
            self.ev_end.synchronize()
            self._device_ms = self.ev_begin.elapsed_time(self.ev_end)
        return self._device_ms / 1e3


class PerfTracer:
    def __init__(self, enabled: bool = True, max_spans: int = 200000):
        self.enabled = enabled
        self._spans: list[Span] = []
        self._lock = threading.Lock()
        self._stack = threading.local()
        self._max = max_spans
        self.t0 = time.perf_counter()

    def _cur(self) -> Optional[Span]:
        st = getattr(self._stack, "s", None)
        return st[-1] if st else None

    @contextlib.contextmanager
    def span(self, name: str, device: bool = False, **tags):
        if not self.enabled:
            yield None
            return
        sp = Span(name, time.perf_counter(), tags=tags, parent=self._cur(),
                  timeline=threading.current_thread().name)
        use_dev = device and torch.cuda.is_available()
        if use_dev:
            sp.ev_begin = torch.cuda.Event(enable_timing=True)
            sp.ev_begin.record()
        if not hasattr(self._stack, "s"):
            self._stack.s = []
        self._stack.s.append(sp)
        try:
            yield sp
        finally:
            if use_dev:
                sp.ev_end = torch.cuda.Event(enable_timing=True)
                sp.ev_end.record()
            sp.end = time.perf_counter()
            self._stack.s.pop()
            with self._lock:
                if len(self._spans) < self._max:
                    self._spans.append(sp)

    def span_group(self, name: str, **tags):
        return self.span(name, device=False, group=True, **tags)

    def spans(self) -> list[Span]:
        with self._lock:
            return list(self._spans)

    def clear(self) -> None:
        with self._lock:
            self._spans.clear()


class NoopTracer(PerfTracer):
    def __init__(self):
        super().__init__(enabled=False)
