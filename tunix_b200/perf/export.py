"""Turn spans of one RL global step into the perf metrics the reference reports
(tunix/perf/export.py:53-569): colocated layout -> perf/global_step_time, perf/weight_sync_time,
perf/{sum,mean}/{rollout_time,refer_inference_time,actor_train_time,actor_train_step_time}; disaggregated
layouts add idle / gap times between micro-batches."""
from __future__ import annotations

from typing import Optional

from .metrics import PerfSpanQuery
from .trace import PerfTracer, Span


def _gaps(spans: list[Span]) -> list[float]:
    spans = sorted(spans, key=lambda s: s.begin)
    return [max(0.0, b.begin - a.end) for a, b in zip(spans, spans[1:]) if a.end is not None]


def export_grpo_metrics(tracer: PerfTracer, step_span: Optional[Span] = None, layout: str = "colocated") -> dict:
    q = PerfSpanQuery.of(tracer)
    if step_span is not None:
        q = q.within(step_span)
    out = {}
    if step_span is not None:
        out["perf/global_step_time"] = step_span.duration
    out["perf/weight_sync_time"] = q.name("weight_sync").total(device=False)
    for key, name in (("rollout_time", "rollout"), ("refer_inference_time", "refer_inference"),
                      ("actor_train_time", "actor_train"), ("actor_train_step_time", "peft_train_step")):
        sel = q.name(name)
        out[f"perf/sum/{key}"] = sel.total()
        out[f"perf/mean/{key}"] = sel.mean()
    if layout in ("rollout_disaggregated", "fully_disaggregated"):
        ro = q.name("rollout").all()
        gaps = _gaps(ro)
        out["perf/rollout_idle_time"] = sum(gaps)
        out["perf/first_micro_batch_rollout_time"] = ro[0].duration if ro else 0.0
        out["perf/sum/between_micro_batch_gap_time"] = sum(gaps)
        out["perf/mean/between_micro_batch_gap_time"] = sum(gaps) / len(gaps) if gaps else 0.0
    if layout == "fully_disaggregated":
        for key, name in (("refer_gap_time", "refer_inference"), ("actor_gap_time", "actor_train")):
            g = _gaps(q.name(name).all())
            out[f"perf/sum/{key}"] = sum(g)
            out[f"perf/mean/{key}"] = sum(g) / len(g) if g else 0.0
    return out
