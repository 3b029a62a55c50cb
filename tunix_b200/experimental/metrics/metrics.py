"""Metrics that stay unreduced until the host asks (tunix/experimental/metrics/metrics.py:22-51).

A `WeightedMetric` is a sum and its weight (a loss summed over tokens and the token count): micro-batches and ranks
add sums and weights, the division happens once. A `MetricsBuffer` carries a step's metrics from a worker to the
orchestrator: weighted ones, plain scalars (lists, reduced by the metric's aggregation function, default mean), and
the mode. Values may be device tensors while the buffer lives on the worker; `to_host()` makes it safe to send."""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Optional, Union

import numpy as np


def _host(v):
    if hasattr(v, "detach"):
        v = v.detach().float().cpu().numpy()
    return np.asarray(v, np.float64)


@dataclasses.dataclass
class WeightedMetric:
    unreduced_sum: Any
    denominator: Any
    eps: Optional[float] = None
    min_denom: Optional[float] = None

    def compute_scale(self):
        d = self.denominator
        if self.eps is not None:
            d = d + self.eps
        if self.min_denom is not None:
            d = d.clamp_min(self.min_denom) if hasattr(d, "clamp_min") else np.maximum(d, self.min_denom)
        return 1.0 / d

    def compute(self):
        return self.unreduced_sum * self.compute_scale()

    def __add__(self, other: "WeightedMetric") -> "WeightedMetric":
        return dataclasses.replace(self, unreduced_sum=self.unreduced_sum + other.unreduced_sum,
                                   denominator=self.denominator + other.denominator)


@dataclasses.dataclass
class MetricsBuffer:
    id: Union[int, str]
    weighted_metrics: Dict[str, WeightedMetric] = dataclasses.field(default_factory=dict)
    scalar_metrics: Dict[str, Any] = dataclasses.field(default_factory=dict)
    aggregation_fns: Dict[str, Callable[[Any], Any]] = dataclasses.field(default_factory=dict)
    mode: str = "train"

    def add_weighted(self, name: str, metric: WeightedMetric) -> None:
        self.weighted_metrics[name] = self.weighted_metrics[name] + metric if name in self.weighted_metrics else metric

    def add_scalar(self, name: str, value, aggregation_fn: Optional[Callable] = None) -> None:
        self.scalar_metrics.setdefault(name, []).append(value)
        if aggregation_fn is not None:
            self.aggregation_fns[name] = aggregation_fn

    def merge(self, other: "MetricsBuffer") -> "MetricsBuffer":
        """Fold another buffer of the same step (another micro-batch, another rank) into this one."""
        for k, m in other.weighted_metrics.items():
            self.add_weighted(k, m)
        for k, vs in other.scalar_metrics.items():
            self.scalar_metrics.setdefault(k, []).extend(vs if isinstance(vs, list) else [vs])
        self.aggregation_fns.update({k: f for k, f in other.aggregation_fns.items() if k not in self.aggregation_fns})
        return self

    def to_host(self) -> "MetricsBuffer":
        return MetricsBuffer(
            self.id, {k: dataclasses.replace(m, unreduced_sum=_host(m.unreduced_sum), denominator=_host(m.denominator))
                      for k, m in self.weighted_metrics.items()},
            {k: [_host(v) for v in (vs if isinstance(vs, list) else [vs])] for k, vs in self.scalar_metrics.items()},
            dict(self.aggregation_fns), self.mode)

    def reduce(self) -> Dict[str, float]:
        """One float per metric (the only place a device value is read)."""
        out = {k: float(_host(m.compute())) for k, m in self.weighted_metrics.items()}
        for k, vs in self.scalar_metrics.items():
            vals = np.asarray([_host(v) for v in (vs if isinstance(vs, list) else [vs])], np.float64)
            out[k] = float(self.aggregation_fns.get(k, np.mean)(vals))
        return out
