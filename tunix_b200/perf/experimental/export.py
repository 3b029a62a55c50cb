"""Export of the step timelines (tunix/perf/experimental/export.py:30-160): a background worker (one thread, so that
writes stay in order) hands the timelines to a trace writer after every step; the training loop never waits for the
file. `from_cluster_config` takes the role → ranks map of the job so that device timelines are grouped by role."""
from __future__ import annotations

import concurrent.futures
import logging
from typing import Any, Mapping, Optional

from . import trace_writer as trace_writer_lib
from .timeline import Timeline

log = logging.getLogger(__name__)
DEFAULT_TRACE_DIR = "/tmp/perf_traces"


def log_metric_export_fn(timelines: Mapping[str, Timeline]) -> dict:
    log.info("\n=== Exporting Timelines ===\n %s", timelines)
    return {}


class PerfMetricsExport:
    @classmethod
    def from_cluster_config(cls, cluster_config, enable_trace_writer: bool = True, trace_dir: Optional[str] = None):
        role_to_devices = {}
        for role, mesh in (getattr(cluster_config, "role_to_mesh", None) or {}).items():
            name = role.value if hasattr(role, "value") else str(role)
            devs = getattr(mesh, "devices", mesh)
            role_to_devices[name] = [int(r) for r in (devs.reshape(-1).tolist() if hasattr(devs, "reshape") else devs)]
        return cls(enable_trace_writer=enable_trace_writer, trace_dir=trace_dir, role_to_devices=role_to_devices)

    def __init__(self, *, enable_trace_writer: bool = True, trace_dir: Optional[str] = None,
                 role_to_devices: Optional[Mapping[str, Any]] = None):
        self._enabled = enable_trace_writer
        if enable_trace_writer:
            self._writer: trace_writer_lib.TraceWriter = trace_writer_lib.PerfettoTraceWriter(trace_dir or DEFAULT_TRACE_DIR,
                                                                                              role_to_devices=role_to_devices)
            self._executor = concurrent.futures.ThreadPoolExecutor(max_workers=1, thread_name_prefix="PerfExport")
        else:
            self._writer = trace_writer_lib.NoopTraceWriter()
            self._executor = None

    @property
    def trace_file_path(self) -> Optional[str]:
        return getattr(self._writer, "trace_file_path", None)

    def _safe_write(self, timelines: Mapping[str, Timeline]) -> None:
        try:
            self._writer.write_timelines(timelines)
        except Exception:
            log.exception("background trace export failed")

    def export_metrics(self, timelines: Mapping[str, Timeline]) -> dict:
        """Queue the timelines for writing; returns no aggregated metrics (the trace is the product)."""
        if self._enabled:
            if self._executor is not None:
                self._executor.submit(self._safe_write, timelines)
            else:
                log.warning("the export worker has been shut down; timelines are not written")
        return {}

    def shutdown(self, wait: bool = True) -> None:
        if self._executor is not None:
            self._executor.shutdown(wait=wait)
            self._executor = None

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.shutdown(wait=True)
