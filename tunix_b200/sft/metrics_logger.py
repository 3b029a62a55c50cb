"""Metric history + fan-out to logging backends (tunix/sft/metrics_logger.py:246-429).

`log(prefix, name, value, mode, step)` records into a per-(prefix, mode, name) history and
forwards scalars to every backend (TensorBoard, W&B offline, JSONL, user factories). Only
rank 0 writes. Perplexity is aggregated as a geometric mean, everything else arithmetically.
"""
from __future__ import annotations

import collections
import json
import os
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


def _is_main_process() -> bool:
    try:
        import torch.distributed as dist
        return (not dist.is_initialized()) or dist.get_rank() == 0
    except Exception:  # pragma: no cover
        return True


class MetricsLogger:
    def __init__(self, metrics_logger_options: Optional[MetricsLoggerOptions] = None, metric_prefix: str = ""):
        self._history: dict = collections.defaultdict(list)
        self._backends: list = []
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
