"""Tagged-span tracer (tunix/perf/experimental/*): spans carry a tag dictionary (step / mini-batch / micro-batch /
role / group / pair) instead of a position in a nesting tree, live on named timelines (one per thread, stream or
asynchronous worker), and are laid out into non-overlapping lanes when written as a Chrome trace.

Device spans take their end from a CUDA event recorded at exit and resolved lazily (`resolve()`), so tracing never
synchronises the stream it measures. Spans submitted from queues that finish out of order are put in sequence per
timeline by `sequentialize` (a span starts no earlier than the end of its predecessor on that timeline)."""
from __future__ import annotations

import contextlib
import dataclasses
import json
import threading
import time
from typing import Optional

import torch


@dataclasses.dataclass
class TaggedSpan:
    name: str
    timeline: str
    begin: float
    end: Optional[float] = None
    tags: dict = dataclasses.field(default_factory=dict)
    _events: Optional[tuple] = None        # (start event, end event, host time at start) for device spans

    @property
    def duration(self) -> Optional[float]:
        return None if self.end is None else self.end - self.begin


class TaggedTracer:
    def __init__(self, enabled: bool = True, clock=time.perf_counter):
        self.enabled, self.clock = enabled, clock
        self._spans: list = []
        self._lock = threading.Lock()
        self._default_tags = threading.local()

    # ------------------------------------------------------------------ tags in scope
    @contextlib.contextmanager
    def tags(self, **tags):
        """Tags applied to every span opened inside this block on the calling thread."""
        prev = getattr(self._default_tags, "v", {})
        self._default_tags.v = {**prev, **tags}
        try:
            yield
        finally:
            self._default_tags.v = prev

    @contextlib.contextmanager
    def span(self, name: str, timeline: Optional[str] = None, device: bool = False, **tags):
        if not self.enabled:
            yield None
            return
        tl = timeline or threading.current_thread().name
        s = TaggedSpan(name, tl, self.clock(), tags={**getattr(self._default_tags, "v", {}), **tags})
        ev = None
        if device and torch.cuda.is_available():
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        try:
            yield s
        finally:
            if ev is not None:
                ev[1].record()
                s._events = (ev[0], ev[1], s.begin)
            s.end = self.clock()
            with self._lock:
                self._spans.append(s)

    def add(self, name: str, timeline: str, begin: float, end: float, **tags) -> TaggedSpan:
        """A span measured elsewhere (an asynchronous worker reporting its own times)."""
        s = TaggedSpan(name, timeline, begin, end, tags)
        with self._lock:
            self._spans.append(s)
        return s

    def resolve(self) -> None:
        """Replace host end times of device spans by device durations, once their events have completed."""
        with self._lock:
            spans = list(self._spans)
        for s in spans:
            if s._events is not None and s._events[1].query():
                s.end = s.begin + s._events[0].elapsed_time(s._events[1]) / 1e3
                s._events = None

    def query(self, name: Optional[str] = None, timeline: Optional[str] = None, **tags) -> list:
        with self._lock:
            spans = list(self._spans)
        return [s for s in spans if (name is None or s.name == name) and (timeline is None or s.timeline == timeline)
                and all(s.tags.get(k) == v for k, v in tags.items())]

    def total(self, name: Optional[str] = None, **tags) -> float:
        return sum(s.duration or 0.0 for s in self.query(name, **tags))

    def clear(self) -> None:
        with self._lock:
            self._spans = []


def sequentialize(spans: list) -> list:
    """Per timeline, in order of begin: a span may not start before its predecessor ended (queued work that was
    timed from submission is shifted to when it could actually run; its duration is kept)."""
    out = []
    by_tl: dict = {}
    for s in sorted(spans, key=lambda s: s.begin):
        by_tl.setdefault(s.timeline, []).append(s)
    for tl, items in by_tl.items():
        t = float("-inf")
        for s in items:
            d = s.duration or 0.0
            b = max(s.begin, t)
            out.append(dataclasses.replace(s, begin=b, end=b + d))
            t = b + d
    return out


def assign_lanes(spans: list) -> dict:
    """Greedy interval colouring per timeline: {id(span): lane}; overlapping spans of a timeline get different lanes."""
    lanes: dict = {}
    by_tl: dict = {}
    for s in spans:
        by_tl.setdefault(s.timeline, []).append(s)
    for items in by_tl.values():
        ends: list = []
        for s in sorted(items, key=lambda s: s.begin):
            for i, e in enumerate(ends):
                if e <= s.begin:
                    ends[i] = s.end if s.end is not None else s.begin
                    lanes[id(s)] = i
                    break
            else:
                ends.append(s.end if s.end is not None else s.begin)
                lanes[id(s)] = len(ends) - 1
    return lanes


def write_chrome_trace(spans: list, path: str) -> None:
    lanes = assign_lanes(spans)
    pids = {tl: i for i, tl in enumerate(sorted({s.timeline for s in spans}))}
    events = [{"name": "process_name", "ph": "M", "pid": pid, "args": {"name": tl}} for tl, pid in pids.items()]
    for s in spans:
        if s.end is None:
            continue
        events.append({"name": s.name, "ph": "X", "pid": pids[s.timeline], "tid": lanes[id(s)], "ts": s.begin * 1e6,
                       "dur": (s.end - s.begin) * 1e6, "args": {k: str(v) for k, v in s.tags.items()}})
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
