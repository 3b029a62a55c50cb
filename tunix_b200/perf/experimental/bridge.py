"""From the spans the always-on tracer recorded to step-organised timelines (the glue the reference has inside its v2
tracer, tunix/perf/experimental/tracer.py): one host timeline per recording thread, one device timeline for the spans
that carry CUDA events (their length is the time between the two events, which is what the GPU spent), committed as one
step. `StepTraceExporter` keeps those timelines across steps and hands them to `PerfMetricsExport` after every step,
which is what `PerfMetricsOptions(enable_perf_v2=True, enable_trace_writer=True, log_dir=...)` switches on in the RL
learners."""
from __future__ import annotations

from typing import Iterable, Mapping, Optional

from . import constants as C
from . import timeline_utils
from .export import PerfMetricsExport
from .timeline import Span, Timeline


def _inside(s, step_span) -> bool:
    if step_span is None:
        return True
    p = s
    while p is not None:
        if p is step_span:
            return True
        p = p.parent
    return s.begin >= step_span.begin and (step_span.end is None or (s.end or s.begin) <= step_span.end)


def add_step(timelines: dict, spans: Iterable, step_span=None, device_id: str = "cuda0", born: Optional[float] = None,
             step: Optional[int] = None) -> dict:
    """Append the spans of one step (those under `step_span`) to `timelines` ({id: Timeline}, created on demand) and commit
    the step on every timeline. Host spans keep their nesting; a span with CUDA events also appears on the device
    timeline with its device duration, placed at its host begin."""
    spans = [s for s in spans if s.end is not None and _inside(s, step_span)]
    born = born if born is not None else min((s.begin for s in spans), default=0.0)
    by_thread: dict = {}
    for s in spans:
        by_thread.setdefault(s.timeline, []).append(s)
    touched = set()
    for thread, group in by_thread.items():
        tl = timelines.setdefault(f"host-{thread}", Timeline(f"host-{thread}", born))
        touched.add(tl.id)
        events = sorted([(s.begin, 1, i, s) for i, s in enumerate(group)] + [(s.end, 0, i, s) for i, s in enumerate(group)],
                        key=lambda e: (e[0], e[1]))
        for t, is_begin, _, s in events:             # replay begin / end in time order: nesting comes out as recorded
            if is_begin:
                tags = {k: v for k, v in s.tags.items() if k != "group"}
                if step is not None:
                    tags.setdefault(C.STEP, step)
                tl.start_span(s.name, t, tags)
            else:
                tl.stop_span(max(t, s.begin))
    dev = [s for s in spans if s.ev_begin is not None and s.ev_end is not None]
    if dev:
        tl = timelines.setdefault(device_id, Timeline(device_id, born))
        touched.add(tl.id)
        for s in sorted(dev, key=lambda x: x.begin):
            d = s.device_duration or 0.0
            tags = dict(s.tags)
            if step is not None:
                tags.setdefault(C.STEP, step)
            tl.start_span(s.name, s.begin, tags)
            tl.stop_span(s.begin + d)
    for tid in touched:
        timelines[tid].commit_step()
    return timelines


class StepTraceExporter:
    def __init__(self, trace_dir: str, role_to_devices: Optional[Mapping] = None, device_id: str = "cuda0"):
        self.timelines: dict = {}
        self.device_id = timeline_utils.generate_device_timeline_id(device_id)
        self._export = PerfMetricsExport(trace_dir=trace_dir, role_to_devices=role_to_devices)
        self._born: Optional[float] = None

    @property
    def trace_file_path(self) -> Optional[str]:
        return self._export.trace_file_path

    def step(self, tracer, step_span, step: Optional[int] = None) -> None:
        """Call once per finished step with the tracer and the step's group span."""
        if self._born is None:
            self._born = getattr(tracer, "t0", None)
        add_step(self.timelines, tracer.spans(), step_span, self.device_id, self._born, step)
        self._export.export_metrics(dict(self.timelines))

    def close(self) -> None:
        self._export.shutdown(wait=True)
