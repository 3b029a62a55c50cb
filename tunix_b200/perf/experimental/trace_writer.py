"""Writers that turn timelines into a trace file (tunix/perf/experimental/trace_writer.py:40-389).

`PerfettoTraceWriter` writes the Chrome / Perfetto JSON trace-event format (ui.perfetto.dev loads it; no protobuf
dependency). Layout: one process per ROLE for device timelines (from `role_to_devices`: {"actor": [0, 1], ...}; a
device that serves several roles appears under each), one process for host timelines, one thread per timeline and
lane. Perfetto wants the slices of a track nested, so spans of a timeline that overlap arbitrarily are spread over
lanes (`_assign_lanes`). Every call rewrites the whole file from the committed steps; failures are logged, never
raised (tracing is best effort)."""
from __future__ import annotations

import abc
import itertools
import json
import logging
import os
import time
from typing import Any, Iterable, Mapping, Optional

from . import constants as C
from . import timeline_utils
from .timeline import Span, Timeline

log = logging.getLogger(__name__)


def _create_span_name(name: str, tags: Mapping[str, Any]) -> str:
    """`name (step=…, group=…)`: the tags that tell two spans of the same name apart, by kind of span."""
    parts = []
    if C.STEP in tags:
        parts.append(f"step={tags[C.STEP]}")
    if name == C.PEFT_TRAIN:
        for key, label in ((C.ROLE, "role"), (C.MINI_BATCH, "mini_batch"), (C.MICRO_BATCH, "micro_batch")):
            if key in tags:
                parts.append(f"{label}={tags[key]}")
    if name in (C.ROLLOUT, C.REFERENCE_INFERENCE, C.OLD_ACTOR_INFERENCE, C.ADVANTAGE_COMPUTATION, C.ENVIRONMENT) and C.GROUP in tags:
        parts.append(f"group_id={tags[C.GROUP]}")
    if name in (C.ROLLOUT, C.ENVIRONMENT) and C.PAIR in tags:
        parts.append(f"pair_index={tags[C.PAIR]}")
    if name == C.QUEUE and C.NAME in tags:
        parts.append(f"name={tags[C.NAME]}")
    return f"{name} ({', '.join(parts)})" if parts else name


def _assign_lanes(spans: Iterable[Span]):
    """({span id: lane}, number of lanes): greedy interval colouring in order of begin."""
    ends: list = []
    lane_of: dict = {}
    for s in sorted(spans, key=lambda x: (x.begin, x.id)):
        for i, e in enumerate(ends):
            if e <= s.begin:
                ends[i], lane_of[s.id] = s.end, i
                break
        else:
            lane_of[s.id] = len(ends)
            ends.append(s.end)
    return lane_of, len(ends)


class TraceWriter(abc.ABC):
    @abc.abstractmethod
    def write_timelines(self, timelines: Mapping[str, Timeline]) -> None:
        ...


class NoopTraceWriter(TraceWriter):
    def write_timelines(self, timelines: Mapping[str, Timeline]) -> None:
        del timelines


class PerfettoTraceWriter(TraceWriter):
    def __init__(self, trace_dir: str, role_to_devices: Optional[Mapping[str, Any]] = None):
        self._role_to_devices = {str(r): timeline_utils.generate_device_timeline_ids(d)
                                 for r, d in (role_to_devices or {}).items()}
        self.trace_file_path: Optional[str] = None
        try:
            os.makedirs(trace_dir, exist_ok=True)
            self.trace_file_path = os.path.join(trace_dir, f"perfetto_trace_v2_{int(time.time())}_{os.getpid()}.json")
        except Exception:
            log.exception("cannot create the trace directory %r; traces are skipped for this run", trace_dir)

    def _tracks_of(self, tl_id: str) -> list:
        """Process names a timeline is shown under."""
        if timeline_utils.is_host_timeline(tl_id):
            return ["host"]
        base = tl_id[:-len("_queue")] if timeline_utils.is_queued_timeline(tl_id) else tl_id
        roles = [r for r, devs in self._role_to_devices.items() if base in devs]
        return [f"role {r}" for r in roles] or ["devices"]

    def write_timelines(self, timelines: Mapping[str, Timeline]) -> None:
        if not timelines or self.trace_file_path is None:
            return
        if not any(any(tl.committed_steps) for tl in timelines.values()):
            return
        try:
            self._write(timelines)
        except Exception:
            log.exception("writing the trace failed")

    def _write(self, timelines: Mapping[str, Timeline]) -> None:
        born = min(tl.born for tl in timelines.values())
        pids: dict = {}
        events: list = []
        next_tid = itertools.count(1)
        for tl_id in sorted(timelines):
            tl = timelines[tl_id]
            spans = list(itertools.chain.from_iterable(step.values() for step in tl.committed_steps))
            if not spans:
                continue
            lane_of, n_lanes = _assign_lanes(spans)
            for track in self._tracks_of(tl_id):
                if track not in pids:
                    pids[track] = len(pids) + 1
                    events.append({"name": "process_name", "ph": "M", "pid": pids[track], "args": {"name": track}})
                tids = [next(next_tid) for _ in range(max(n_lanes, 1))]
                for lane, tid in enumerate(tids):
                    events.append({"name": "thread_name", "ph": "M", "pid": pids[track], "tid": tid,
                                   "args": {"name": tl_id if lane == 0 else f"{tl_id} +{lane}"}})
                for s in spans:
                    if not s.ended:
                        continue
                    events.append({"name": _create_span_name(s.name, s.tags), "ph": "X", "pid": pids[track],
                                   "tid": tids[lane_of[s.id]], "ts": (s.begin - born) * 1e6, "dur": s.duration * 1e6,
                                   "args": {str(k): str(v) for k, v in s.tags.items()}})
        tmp = self.trace_file_path + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
        os.replace(tmp, self.trace_file_path)
