"""Write spans as a Chrome / Perfetto trace (JSON trace-event format, loadable in ui.perfetto.dev)
(role of tunix/perf/perfetto.py:152-230; the JSON encoding needs no protobuf dependency)."""
from __future__ import annotations

import json
import os

from .trace import PerfTracer


def write_trace(tracer: PerfTracer, path: str, process_name: str = "tunix_b200") -> str:
    events = [{"name": "process_name", "ph": "M", "pid": 0, "args": {"name": process_name}}]
    tids: dict = {}
    for s in tracer.spans():
        tid = tids.setdefault(s.timeline, len(tids))
        ev = {"name": s.name, "ph": "X", "pid": 0, "tid": tid, "ts": (s.begin - tracer.t0) * 1e6,
              "dur": s.duration * 1e6, "args": {k: v for k, v in s.tags.items()}}
        events.append(ev)
        d = s.device_duration
        if d is not None:
            dtid = tids.setdefault(s.timeline + "/device", len(tids))
            events.append({"name": s.name, "ph": "X", "pid": 0, "tid": dtid, "ts": (s.begin - tracer.t0) * 1e6,
                           "dur": d * 1e6, "args": {"device": True}})
    for name, tid in tids.items():
        events.append({"name": "thread_name", "ph": "M", "pid": 0, "tid": tid, "args": {"name": name}})
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
    return path
