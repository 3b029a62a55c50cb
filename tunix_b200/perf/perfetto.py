"""Write spans as a Chrome / Perfetto trace (JSON trace-event format, loadable in ui.perfetto.dev)
(role of tunix/perf/perfetto.py:152-230; the JSON encoding needs no protobuf dependency)."""
from __future__ import annotations

import json
import os

from .trace import PerfTracer


def write_trace(tracer: PerfTracer, path: str, process_name: str = "tunix_b200") -> str:
    return write_spans(tracer.spans(), path, tracer.t0, process_name)


def write_spans(spans: list, path: str, t0: float = 0.0, process_name: str = "tunix_b200") -> str:
    """The same file from a list of spans (one global step, one rank): what the metrics exporters write per step."""
    class _T:
        pass
    tracer = _T()
    tracer.t0 = t0
    events = [{"name": "process_name", "ph": "M", "pid": 0, "args": {"name": process_name}}]
    tids: dict = {}
    for s in spans:
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
