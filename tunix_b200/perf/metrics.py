"""Span queries (tunix/perf/metrics.py:133-227)."""
from __future__ import annotations

from typing import Callable, Optional

from .trace import PerfTracer, Span


class PerfSpanQuery:
    def __init__(self, spans: list[Span]):
        self._spans = spans

    @classmethod
    def of(cls, tracer: PerfTracer) -> "PerfSpanQuery":
        return cls(tracer.spans())

    def name(self, name: str) -> "PerfSpanQuery":
        return PerfSpanQuery([s for s in self._spans if s.name == name])

    def tag(self, **tags) -> "PerfSpanQuery":
        return PerfSpanQuery([s for s in self._spans if all(s.tags.get(k) == v for k, v in tags.items())])

    def within(self, parent: Span) -> "PerfSpanQuery":
        def inside(s):
            p = s.parent
            while p is not None:
                if p is parent:
                    return True
                p = p.parent
            return False
        return PerfSpanQuery([s for s in self._spans if inside(s)])

    def where(self, pred: Callable[[Span], bool]) -> "PerfSpanQuery":
        return PerfSpanQuery([s for s in self._spans if pred(s)])

    def all(self) -> list[Span]:
        return list(self._spans)

    def total(self, device: bool = True) -> float:
        tot = 0.0
        for s in self._spans:
            d = s.device_duration if device else None
            tot += d if d is not None else s.duration
        return tot

    def mean(self, device: bool = True) -> float:
        return self.total(device) / len(self._spans) if self._spans else 0.0

    def count(self) -> int:
        return len(self._spans)
