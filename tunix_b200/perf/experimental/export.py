"""Export of the step timelines (tunix/perf/experimental/export.py:30-160): after every step the timelines go to a
trace writer on a worker thread of their own, so that the training loop never waits for a file and writes stay in
order. `from_cluster_config` reads the job's role → ranks map, which the writer uses to group device timelines."""
from __future__ import annotations

import logging
import queue
import threading
from typing import Any, Mapping, Optional

from . import trace_writer as trace_writer_lib
from .timeline import Timeline

log = logging.getLogger(__name__)
DEFAULT_TRACE_DIR = "/tmp/perf_traces"
_STOP = object()


def log_metric_export_fn(timelines: Mapping[str, Timeline]) -> dict:
    log.info("\n=== Exporting Timelines ===\n %s", timelines)
    return {}


def _ranks_of(mesh) -> list:
    devices = getattr(mesh, "devices", mesh)
    flat = devices.reshape(-1).tolist() if hasattr(devices, "reshape") else list(devices)
    return [int(r) for r in flat]


class PerfMetricsExport:
    def __init__(self, *, enable_trace_writer: bool = True, trace_dir: Optional[str] = None,
                 role_to_devices: Optional[Mapping[str, Any]] = None):
        self._jobs: Optional["queue.Queue"] = None
        self._thread: Optional[threading.Thread] = None
        if not enable_trace_writer:
            self._writer: trace_writer_lib.TraceWriter = trace_writer_lib.NoopTraceWriter()
            return
        self._writer = trace_writer_lib.PerfettoTraceWriter(trace_dir or DEFAULT_TRACE_DIR, role_to_devices=role_to_devices)
        self._jobs = queue.Queue()
        self._thread = threading.Thread(target=self._drain, name="PerfExport", daemon=True)
        self._thread.start()

    @classmethod
    def from_cluster_config(cls, cluster_config, enable_trace_writer: bool = True, trace_dir: Optional[str] = None):
        meshes = getattr(cluster_config, "role_to_mesh", None) or {}
        roles = {getattr(role, "value", str(role)): _ranks_of(mesh) for role, mesh in meshes.items() if mesh is not None}
        return cls(enable_trace_writer=enable_trace_writer, trace_dir=trace_dir, role_to_devices=roles)

    @property
    def trace_file_path(self) -> Optional[str]:
        return getattr(self._writer, "trace_file_path", None)

    def _drain(self) -> None:
        while True:
            job = self._jobs.get()
            if job is _STOP:
                return
            try:
                self._writer.write_timelines(job)
            except Exception:                      # tracing is best effort
                log.exception("background trace export failed")

    def export_metrics(self, timelines: Mapping[str, Timeline]) -> dict:
        """Queue the timelines for writing; there are no aggregated metrics to return (the trace is the product)."""
        if self._jobs is not None:
            if self._thread is not None and self._thread.is_alive():
                self._jobs.put(timelines)
            else:
                log.warning("the export worker has been shut down; timelines are not written")
        return {}

    def shutdown(self, wait: bool = True) -> None:
        if self._thread is None:
            return
        self._jobs.put(_STOP)
        if wait:
            self._thread.join()
        self._thread = None

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.shutdown(wait=True)
