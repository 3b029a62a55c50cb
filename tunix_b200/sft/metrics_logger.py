"""Metric history + fan-out to logging backends (tunix/sft/metrics_logger.py:246-429).

`log(prefix, name, value, mode, step)` records into a per-(prefix, mode, name) history and
forwards scalars to every backend (TensorBoard, W&B offline, JSONL, user factories). Only
rank 0 writes. Perplexity is aggregated as a geometric mean, everything else arithmetically.

With `enable_opentelemetry` every scalar is also set on a synchronous OpenTelemetry gauge (`:331-381`): instrument
`tunix.training.<name>` for the known training metrics, `tunix.<normalised name>` otherwise; prefix and mode travel
as attributes; the logical step is a gauge of its own (`tunix.training.step`), because a step attribute would make a
new time series per step. `sft.otel_wandb.WandbMetricsExporter` turns those gauges into W&B log calls.
"""
from __future__ import annotations

import collections
import json
import logging
import os
import re
import threading
import time
from typing import Any, Callable, Optional, Protocol

import numpy as np

from ..common.configs import MetricsLoggerOptions
from ..common.datatypes import Mode


class LoggingBackend(Protocol):
    def log_scalar(self, event: str, value: float, **kwargs) -> None: ...
    def close(self) -> None: ...


class JsonlBackend:
    def __init__(self, log_dir: str):
        os.makedirs(log_dir, exist_ok=True)
        self._f = open(os.path.join(log_dir, "metrics.jsonl"), "a")
        self._lock = threading.Lock()

    def log_scalar(self, event: str, value: float, **kwargs) -> None:
        rec = {"event": event, "value": float(value), "step": kwargs.get("step"), "time": time.time()}
        with self._lock:
            self._f.write(json.dumps(rec) + "\n")

    def flush(self):
        with self._lock:
            self._f.flush()

    def close(self) -> None:
        with self._lock:
            self._f.close()


class TensorboardBackend:
    def __init__(self, log_dir: str, flush_every_n_steps: int = 100):
        from torch.utils.tensorboard import SummaryWriter
        self._w = SummaryWriter(log_dir=log_dir, max_queue=flush_every_n_steps)

    def log_scalar(self, event: str, value: float, **kwargs) -> None:
        self._w.add_scalar(event, float(value), kwargs.get("step"))

    def close(self) -> None:
        self._w.close()


class WandbBackend:
    def __init__(self, project: str, name: str = ""):
        import wandb
        os.environ.setdefault("WANDB_MODE", "offline")
        self._run = wandb.init(project=project, name=name or None, reinit=True)

    def log_scalar(self, event: str, value: float, **kwargs) -> None:
        self._run.log({event: float(value)}, step=kwargs.get("step"))

    def close(self) -> None:
        self._run.finish()


OTEL_STEP_METRIC = "tunix.training.step"
OTEL_PREFIX_ATTRIBUTE = "tunix.metrics.prefix"
OTEL_MODE_ATTRIBUTE = "tunix.training.mode"
_OTEL_KNOWN = {"loss": "tunix.training.loss", "perplexity": "tunix.training.perplexity",
               "learning_rate": "tunix.training.learning_rate", "grad_norm": "tunix.training.grad_norm",
               "step_time_sec": "tunix.training.step_time", "tflops_per_step": "tunix.training.tflops_per_step"}


def otel_metric_name(metric_name: str) -> str:
    """A valid, namespaced instrument name: known training metrics keep a stable name, anything else becomes
    `tunix.<name with runs of other characters replaced by dots, lower case>`."""
    if metric_name in _OTEL_KNOWN:
        return _OTEL_KNOWN[metric_name]
    norm = re.sub(r"[^a-zA-Z0-9_.-]+", ".", metric_name).strip(".") or "unnamed"
    return f"tunix.{norm.lower()}"


class OtelGaugeEmitter:
    def __init__(self, meter_provider=None):
        from opentelemetry import metrics as otel_metrics
        provider = meter_provider if meter_provider is not None else otel_metrics.get_meter_provider()
        self._meter = provider.get_meter("tunix_b200")
        self._gauges: dict = {}
        self._last_step: dict = {}
        self._lock = threading.Lock()

    def _gauge(self, name: str, unit: str = "1"):
        with self._lock:
            g = self._gauges.get(name)
            if g is None:
                g = self._gauges[name] = self._meter.create_gauge(name, unit=unit)
            return g

    def emit(self, prefix: str, metric_name: str, value: float, mode, step: Optional[int]) -> None:
        attrs = {OTEL_MODE_ATTRIBUTE: str(mode)}
        if prefix:
            attrs[OTEL_PREFIX_ATTRIBUTE] = prefix
        self._gauge(otel_metric_name(metric_name)).set(value, attrs)
        if step is None:
            return
        with self._lock:
            if self._last_step.get((prefix, str(mode))) == step:
                return
            self._last_step[(prefix, str(mode))] = step
        self._gauge(OTEL_STEP_METRIC, "{step}").set(int(step), attrs)


def _is_main_process() -> bool:
    try:
        import torch.distributed as dist
        return (not dist.is_initialized()) or dist.get_rank() == 0
    except Exception:  # pragma: no cover
        return True


class MetricsLogger:
    def __init__(self, metrics_logger_options: Optional[MetricsLoggerOptions] = None, metric_prefix: str = "",
                 otel_meter_provider=None):
        self._history: dict = collections.defaultdict(list)
        self._backends: list = []
        self._otel: Optional[OtelGaugeEmitter] = None
        if metrics_logger_options is not None and getattr(metrics_logger_options, "enable_opentelemetry", False) \
                and _is_main_process():
            try:
                self._otel = OtelGaugeEmitter(otel_meter_provider)
            except ImportError:
                logging.getLogger(__name__).warning("enable_opentelemetry is set but the opentelemetry package is missing")
        self._prefix = metric_prefix
        self._lock = threading.Lock()
        opts = metrics_logger_options
        if opts is not None and _is_main_process():
            if opts.backend_factories:
                for fac in opts.backend_factories:
                    if not callable(fac):
                        raise TypeError("backend_factories entries must be callables returning a backend")
                    self._backends.append(fac())
            elif opts.log_dir:
                if opts.use_jsonl:
                    self._backends.append(JsonlBackend(opts.log_dir))
                if opts.use_tensorboard:
                    try:
                        self._backends.append(TensorboardBackend(opts.log_dir, opts.flush_every_n_steps))
                    except Exception:  # tensorboard missing
                        pass
                if opts.use_wandb:
                    try:
                        self._backends.append(WandbBackend(opts.project_name, opts.run_name))
                    except Exception:
                        pass

    @staticmethod
    def _key(prefix: str, name: str, mode) -> str:
        mode = str(mode)
        return f"{prefix}/{mode}/{name}" if prefix else f"{mode}/{name}"

    def log(self, metrics_prefix: str, metric_name: str, scalar_value: Any, mode=Mode.TRAIN, step: Optional[int] = None):
        try:
            v = float(np.asarray(scalar_value.detach().cpu() if hasattr(scalar_value, "detach") else scalar_value).reshape(()))
        except Exception:
            return
        key = self._key(metrics_prefix, metric_name, mode)
        with self._lock:
            self._history[key].append(v)
        for b in self._backends:
            b.log_scalar(key, v, step=step)
        if self._otel is not None:
            try:
                self._otel.emit(metrics_prefix, metric_name, v, mode, step)
            except Exception:                       # telemetry never takes a training step down
                logging.getLogger(__name__).exception("failed to emit OpenTelemetry metric %s", key)

    def metric_exists(self, metrics_prefix: str, metric_name: str, mode) -> bool:
        return len(self._history.get(self._key(metrics_prefix, metric_name, mode), ())) > 0

    def get_metric(self, metrics_prefix: str, metric_name: str, mode):
        key = self._key(metrics_prefix, metric_name, mode)
        vals = self._history.get(key)
        if not vals:
            raise ValueError(f"metric {key} not found")
        arr = np.asarray(vals, dtype=np.float64)
        if metric_name == "perplexity":
            return float(np.exp(np.mean(np.log(np.maximum(arr, 1e-30)))))
        return float(arr.mean())

    def get_metric_history(self, metrics_prefix: str, metric_name: str, mode):
        return np.asarray(self._history.get(self._key(metrics_prefix, metric_name, mode), []))

    def close(self):
        for b in self._backends:
            try:
                b.close()
            except Exception:  # pragma: no cover
                pass
        self._backends = []
