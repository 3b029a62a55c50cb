"""Timelines of spans, organised in steps (tunix/perf/experimental/timeline.py:30-410).

A `Timeline` records spans on one logical lane (the host thread of a role, a CUDA stream, a queue). Synchronous spans
nest through a stack (`start_span` / `stop_span`); `commit_step` closes the current step: its finished spans become an
immutable entry of `committed_steps` (readers need no lock), spans still open are purged with a warning.

`AsyncTimeline.span(name, begin, waitlist)` records a leaf span that ends when device work has finished, without
blocking the caller. `waitlist` is what marks that point on this hardware: a `torch.cuda.Event` (or several), a
tensor (an event is recorded on the current stream at the call), a `concurrent.futures.Future`, or nothing (the span
ends at once). A watcher thread waits (`event.synchronize()` blocks that thread only) and stamps the end time.
`BatchAsyncTimelines` records the same span on several timelines (one per GPU of a role) with ONE watcher.
"""
from __future__ import annotations

import concurrent.futures as futures
import dataclasses
import logging
import threading
import time
from typing import Any, Callable, Mapping, Optional

log = logging.getLogger(__name__)
_INF = float("inf")


@dataclasses.dataclass
class Span:
    name: str
    begin: float
    id: int
    end: float = dataclasses.field(default=_INF, init=False)
    parent_id: Optional[int] = None
    tags: Optional[Mapping[str, Any]] = None

    def __post_init__(self) -> None:
        self.tags = dict(self.tags) if self.tags is not None else {}

    def add_tag(self, key: str, value: Any) -> None:
        if key in self.tags:
            log.warning("span %r (id=%s): tag %r already holds %r, overwriting with %r", self.name, self.id, key,
                        self.tags[key], value)
        self.tags[key] = value

    def _format_relative(self, born_at: float) -> str:
        out = f"[{self.id}] {self.name}: {self.begin - born_at:.6f}, {self.end - born_at:.6f}"
        if self.parent_id is not None:
            out += f" (parent={self.parent_id})"
        if self.tags:
            out += f", tags={self.tags}"
        return out

    @property
    def ended(self) -> bool:
        return self.end != _INF

    @property
    def duration(self) -> float:
        return self.end - self.begin


class Timeline:
    def __init__(self, id: str, born: float):
        self.id, self.born = id, born
        self._spans_stack: list = []
        self._cur_step: dict = {}
        self._last_span_id = -1
        self._committed_steps: list = []
        self._lock = threading.RLock()

    @property
    def committed_steps(self) -> list:
        """Committed steps ({span id: Span} each); the list is replaced, never mutated, so reading needs no lock."""
        return self._committed_steps

    @property
    def cur_step(self) -> dict:
        with self._lock:
            return dict(self._cur_step)

    @property
    def all_steps(self) -> list:
        with self._lock:
            return self._committed_steps + [dict(self._cur_step)]

    def start_span(self, name: str, begin: float, tags: Optional[Mapping[str, Any]] = None) -> Span:
        with self._lock:
            parent = self._spans_stack[-1] if self._spans_stack else None
            self._last_span_id += 1
            s = Span(name=name, begin=begin, id=self._last_span_id, parent_id=parent, tags=tags)
            self._cur_step[s.id] = s
            self._spans_stack.append(s.id)
        return s

    def stop_span(self, end: float) -> None:
        with self._lock:
            if not self._spans_stack:
                raise ValueError(f"{self.id}: no more spans to end.")
            s = self._cur_step[self._spans_stack.pop()]
            if s.begin > end:
                raise ValueError(f"{self.id}: span '{s.name}' ended at {end:.6f} before it began at {s.begin:.6f}.")
            s.end = end

    def commit_step(self) -> None:
        with self._lock:
            for sid in [sid for sid, s in self._cur_step.items() if not s.ended or sid in self._spans_stack]:
                log.warning("purging unfinished span %r that crosses a step boundary of timeline %s",
                            self._cur_step[sid].name, self.id)
                self._cur_step.pop(sid, None)
            self._spans_stack.clear()
            self._committed_steps = list(self._committed_steps) + [self._cur_step]      # copy on write
            self._cur_step = {}

    def __repr__(self) -> str:
        parts = [f"Timeline({self.id}, {self.born:.6f})\n"]
        with self._lock:
            if self._cur_step:
                parts.append(f"Current Step -{len(self._committed_steps)}:\n")
                parts += [f"  {s._format_relative(self.born)}\n" for s in sorted(self._cur_step.values(), key=lambda s: s.id)]
            for i, step in enumerate(reversed(self._committed_steps)):
                if step:
                    parts.append(f"Committed Step -{i}:\n")
                    parts += [f"  {s._format_relative(self.born)}\n" for s in sorted(step.values(), key=lambda s: s.id)]
        return "".join(parts)


def _flatten(waitlist) -> list:
    if waitlist is None:
        return []
    if isinstance(waitlist, (list, tuple)):
        return [w for x in waitlist for w in _flatten(x)]
    if isinstance(waitlist, dict):
        return [w for x in waitlist.values() for w in _flatten(x)]
    return [waitlist]


def _to_waitables(waitlist) -> list:
    """Things a watcher thread can block on: CUDA events (a tensor is replaced by an event recorded now on the
    current stream of its device), futures, objects with `wait()` / `synchronize()`."""
    out = []
    for w in _flatten(waitlist):
        try:
            import torch
            if isinstance(w, torch.Tensor):
                if w.is_cuda:
                    ev = torch.cuda.Event()
                    ev.record(torch.cuda.current_stream(w.device))
                    out.append(ev)
                continue
        except ImportError:       # pragma: no cover
            pass
        out.append(w)
    return out


def _wait_one(w) -> None:
    if isinstance(w, futures.Future):
        w.result()
    elif hasattr(w, "synchronize"):
        w.synchronize()
    elif hasattr(w, "wait"):
        w.wait()
    else:
        raise TypeError(f"cannot wait on {type(w).__name__}")


def _async_wait(waitables: list, success: Callable[[], None], failure: Callable[[Exception], None]) -> threading.Thread:
    def run():
        try:
            for w in waitables:
                _wait_one(w)
        except Exception as e:  # metrics are best effort
            failure(e)
            return
        success()
    t = threading.Thread(target=run, daemon=True, name="timeline-wait")
    t.start()
    return t


class AsyncTimeline(Timeline):
    """A timeline whose spans close when device work (or a future) completes."""

    def __init__(self, id: str, born: float):
        super().__init__(id, born)
        self._threads: list = []

    def _reserve(self):
        with self._lock:
            parent = self._spans_stack[-1] if self._spans_stack else None
            self._last_span_id += 1
            return self._last_span_id, parent

    def _finish(self, span_id: int, parent, name: str, begin: float, end: float, tags) -> None:
        with self._lock:
            s = Span(name=name, begin=begin, id=span_id, parent_id=parent, tags=tags)
            s.end = end
            self._cur_step[span_id] = s

    def span(self, name: str, thread_span_begin: float, waitlist=None, tags: Optional[Mapping[str, Any]] = None) -> None:
        """A leaf span from `thread_span_begin` (a `time.perf_counter()` value of the caller) to the moment everything
        in `waitlist` has completed. Asynchronous spans are never parents."""
        span_id, parent = self._reserve()
        waitables = _to_waitables(waitlist)

        def ok():
            self._finish(span_id, parent, name, thread_span_begin, time.perf_counter(), tags)

        def bad(e):
            log.error("timeline span %r (id=%d) failed: %s", name, span_id, e)
        if not waitables:
            ok()
            return
        t = _async_wait(waitables, ok, bad)
        with self._lock:
            self._threads = [x for x in self._threads if x.is_alive()] + [t]

    def wait_pending_spans(self) -> None:
        with self._lock:
            cur, self._threads = list(self._threads), []
        for t in cur:
            t.join()


class BatchAsyncTimelines:
    """The same asynchronous span on several timelines (the GPUs of a role), closed by one watcher thread."""

    def __init__(self, timelines: list):
        self._timelines = list(timelines)
        self._threads: list = []

    def span(self, name: str, thread_span_begin: float, waitlist=None, tags: Optional[Mapping[str, Any]] = None) -> None:
        reserved = [(tl, *tl._reserve()) for tl in self._timelines]
        waitables = _to_waitables(waitlist)

        def ok():
            end = time.perf_counter()
            for tl, sid, parent in reserved:
                tl._finish(sid, parent, name, thread_span_begin, end, tags)

        def bad(e):
            log.error("timeline span %r failed: %s", name, e)
        if not waitables:
            ok()
            return
        self._threads = [x for x in self._threads if x.is_alive()] + [_async_wait(waitables, ok, bad)]

    def wait_pending_spans(self) -> None:
        cur, self._threads = list(self._threads), []
        for t in cur:
            t.join()
