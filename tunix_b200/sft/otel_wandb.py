"""OpenTelemetry metric exporter that logs to a Weights & Biases run (tunix/sft/otel_wandb.py:45-157).

W&B has no OTLP endpoint for run metrics; this exporter closes the gap for the gauges that
`sft.metrics_logger.MetricsLogger` writes with `enable_opentelemetry`:

    reader = PeriodicExportingMetricReader(WandbMetricsExporter(run), export_interval_millis=10_000)
    logger = MetricsLogger(MetricsLoggerOptions(log_dir=..., enable_opentelemetry=True),
                           otel_meter_provider=MeterProvider(metric_readers=[reader]))

Data points are grouped by (prefix, mode); the group's `tunix.training.step` gauge gives the W&B step of the other
values; chart keys are `<prefix>/<mode>/<instrument>`; groups are logged in ascending step order (W&B refuses a step
that goes backwards). The run is not finished on shutdown: whoever called `wandb.init` owns it."""
from __future__ import annotations

import logging
from typing import Any, Iterator, Optional, Tuple

from opentelemetry.sdk.metrics import export as otel_export

from .metrics_logger import OTEL_MODE_ATTRIBUTE, OTEL_PREFIX_ATTRIBUTE, OTEL_STEP_METRIC

log = logging.getLogger(__name__)


def _wandb_key(prefix: str, mode: str, metric_name: str) -> str:
    return "/".join(p for p in (prefix, mode, metric_name) if p)


def _points(metrics_data):
    """(prefix, mode, instrument name, value) of every data point in an export batch."""
    for resource in metrics_data.resource_metrics:
        for scope in resource.scope_metrics:
            for metric in scope.metrics:
                for point in getattr(metric.data, "data_points", ()):
                    attrs = point.attributes or {}
                    yield str(attrs.get(OTEL_PREFIX_ATTRIBUTE, "")), str(attrs.get(OTEL_MODE_ATTRIBUTE, "")), metric.name, point.value


def _wandb_payloads(metrics_data) -> Iterator[Tuple[Optional[int], dict]]:
    """(step, {chart key: value}) per (prefix, mode) group, in ascending step order; groups without a step gauge come
    last with step None."""
    steps: dict = {}
    values: dict = {}
    for prefix, mode, name, value in _points(metrics_data):
        if name == OTEL_STEP_METRIC:
            steps[(prefix, mode)] = int(value)
        else:
            values.setdefault((prefix, mode), {})[_wandb_key(prefix, mode, name)] = value
    order = sorted(values, key=lambda g: (g not in steps, steps.get(g, 0)))
    for group in order:
        yield steps.get(group), values[group]


class WandbMetricsExporter(otel_export.MetricExporter):
    def __init__(self, run: Any = None, **kwargs):
        """`run`: what `wandb.init` returned; None resolves the global `wandb.run` at export time."""
        super().__init__(**kwargs)
        self._run = run

    def _resolve_run(self):
        if self._run is not None:
            return self._run
        import wandb
        if wandb.run is None:
            raise RuntimeError("WandbMetricsExporter has no W&B run to log to. Pass a run to the exporter or call wandb.init() "
                               "before exporting.")
        return wandb.run

    def export(self, metrics_data, timeout_millis: float = 10_000, **kwargs):
        try:
            run = self._resolve_run()
            for step, values in _wandb_payloads(metrics_data):
                run.log(values, step=step)
        except Exception:
            log.exception("Failed to export OpenTelemetry metrics to W&B.")
            return otel_export.MetricExportResult.FAILURE
        return otel_export.MetricExportResult.SUCCESS

    def force_flush(self, timeout_millis: float = 10_000) -> bool:
        return True

    def shutdown(self, timeout_millis: float = 30_000, **kwargs) -> None:
        pass
