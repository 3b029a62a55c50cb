"""Spans of one RL global step -> the perf metrics the reference reports, per layout
(tunix/perf/export.py:53-569).

The reference picks one of three GRPO exporters from the role -> devices map: everything on one mesh; rollout on
one mesh and actor + reference on another; three different meshes (`from_role_to_devices`, :75-125;
`from_cluster_config`, :127-190). The same selection is made here from role -> ranks:

    colocated                 perf/global_step_time, perf/weight_sync_time,
                              perf/{sum,mean}/{rollout,refer_inference,actor_train,actor_train_step}_time
    rollout | actor+refer     + perf/rollout_idle_time (end of the last rollout -> start of the weight sync),
                              perf/first_micro_batch_rollout_time (step start -> first rollout result),
                              perf/{sum,mean}/between_micro_batch_gap_time (end of an actor update -> start of the next
                              reference scoring)
    rollout | actor | refer   + perf/{sum,mean}/refer_gap_time and actor_gap_time (begin of one span -> end of the next)

One process per GPU means that a rank only sees its own spans. What a rank cannot see (a controller does not see the
sampler's kernel time, a serving rank does not see the updates) is simply absent from its dictionary;
`merge_over_ranks` puts the dictionaries of all ranks together (max for step-level times, the serving ranks' figures
under `perf/<role>/...`). The span names are the ones `RLCluster` and the trainers record: `global_step` (group),
`rollout`, `refer_inference`, `actor_train`, `peft_train_step`, `weight_sync`.
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np

from .metrics import PerfSpanQuery
from .trace import PerfTracer, Span

COLOCATED, ROLLOUT_APART, FULLY_APART = "colocated", "rollout_disaggregated", "fully_disaggregated"


def _dur(s: Span) -> float:
    d = s.device_duration
    return d if d is not None else s.duration


def _stats(out: dict, key: str, values: list) -> None:
    out[f"perf/sum/{key}"] = float(np.sum(values)) if values else 0.0
    out[f"perf/mean/{key}"] = float(np.mean(values)) if values else 0.0


def layout_of(role_to_ranks: dict) -> str:
    """The reference's three cases from {"rollout": [...], "actor": [...], "refer": [...]} (:98-117)."""
    ro, ac, rf = (sorted(role_to_ranks[k]) for k in ("rollout", "actor", "refer"))
    if ro == ac == rf:
        return COLOCATED
    if ro != ac and ac == rf:
        return ROLLOUT_APART
    if ro != ac and ac != rf:
        return FULLY_APART
    raise ValueError("unsupported placement for the perf metrics: rollout and actor share their ranks but the reference "
                     "has others")


def _step_spans(q: PerfSpanQuery, step_span: Optional[Span]):
    """(step span, query restricted to it): the given one, else the last `global_step` group on record."""
    if step_span is None:
        groups = [s for s in q.name("global_step").all() if s.end is not None]
        step_span = max(groups, key=lambda s: s.begin) if groups else None
    if step_span is None:
        return None, q
    inner = q.within(step_span)
    # spans of other threads (the rollout producer) have no parent on this thread: they belong to the step whose
    # time window holds them
    end = step_span.end if step_span.end is not None else float("inf")
    have = {id(s) for s in inner.all()}

    def root(s):
        while s.parent is not None:
            s = s.parent
        return s
    extra = [s for s in q.all() if id(s) not in have and s is not step_span and root(s).timeline != step_span.timeline
             and root(s).name != "global_step" and step_span.begin <= s.begin and (s.end or s.begin) <= end]
    return step_span, PerfSpanQuery(inner.all() + extra)


def _common(q: PerfSpanQuery, step: Optional[Span]) -> tuple:
    by = lambda name: sorted(q.name(name).all(), key=lambda s: s.begin)  # noqa: E731
    rollout, refer, train, train_steps = by("rollout"), by("refer_inference"), by("actor_train"), by("peft_train_step")
    syncs = by("weight_sync")
    out = {}
    if step is not None:
        out["perf/global_step_time"] = step.duration
    out["perf/weight_sync_time"] = syncs[-1].duration if syncs else 0.0     # a shared model never syncs: zero
    _stats(out, "rollout_time", [_dur(s) for s in rollout])
    _stats(out, "refer_inference_time", [_dur(s) for s in refer])
    _stats(out, "actor_train_time", [_dur(s) for s in train])
    _stats(out, "actor_train_step_time", [_dur(s) for s in train_steps])
    return out, rollout, refer, train, (syncs[-1] if syncs else None)


def grpo_metrics_colocated(q: PerfSpanQuery, step_span: Optional[Span] = None) -> dict:
    step, q = _step_spans(q, step_span)
    return _common(q, step)[0]


def grpo_metrics_rollout_apart(q: PerfSpanQuery, step_span: Optional[Span] = None) -> dict:
    step, q = _step_spans(q, step_span)
    out, rollout, refer, train, sync = _common(q, step)
    if rollout:
        end_ref = sync.begin if sync is not None else (step.end if step is not None and step.end else rollout[-1].end)
        out["perf/rollout_idle_time"] = max(0.0, end_ref - rollout[-1].end)
        out["perf/first_micro_batch_rollout_time"] = rollout[0].end - (step.begin if step is not None else rollout[0].begin)
    gaps = [max(0.0, b.begin - a.end) for a, b in zip(train[:-1], refer[1:])] + [0.0]   # one entry per micro-batch
    _stats(out, "between_micro_batch_gap_time", gaps if train else [])
    return out


def grpo_metrics_fully_apart(q: PerfSpanQuery, step_span: Optional[Span] = None) -> dict:
    step, q = _step_spans(q, step_span)
    out, rollout, refer, train, sync = _common(q, step)
    if rollout:
        end_ref = sync.begin if sync is not None else (step.end if step is not None and step.end else rollout[-1].end)
        out["perf/rollout_idle_time"] = max(0.0, end_ref - rollout[-1].end)
        out["perf/first_micro_batch_rollout_time"] = rollout[0].end - (step.begin if step is not None else rollout[0].begin)
    _stats(out, "refer_gap_time", ([b.end - a.begin for a, b in zip(refer[:-1], refer[1:])] + [0.0]) if refer else [])
    _stats(out, "actor_gap_time", ([b.end - a.begin for a, b in zip(train[:-1], train[1:])] + [0.0]) if train else [])
    return out


_EXPORTERS = {COLOCATED: grpo_metrics_colocated, ROLLOUT_APART: grpo_metrics_rollout_apart,
              FULLY_APART: grpo_metrics_fully_apart}


class PerfMetricsExport:
    """Factories for `export_fn(query_or_tracer[, step_span]) -> {metric: seconds}`."""

    @staticmethod
    def from_role_to_ranks(role_to_ranks: dict, trace_writer=None) -> Callable:
        fn = _EXPORTERS[layout_of(role_to_ranks)]

        def export(source, step_span: Optional[Span] = None) -> dict:
            q = PerfSpanQuery.of(source) if isinstance(source, PerfTracer) else source
            out = fn(q, step_span)
            if trace_writer is not None:
                step, inner = _step_spans(q, step_span)
                trace_writer(([step] if step is not None else []) + inner.all())
            return out
        export.layout = layout_of(role_to_ranks)
        return export

    from_role_to_devices = from_role_to_ranks      # the reference's name; devices are ranks here

    @staticmethod
    def from_cluster_config(cluster_config, placement=None) -> Callable:
        """Layout from `cluster_config.role_to_mesh` (or an already built `RolePlacement`); a Chrome-trace writer is
        attached when `training_config.perf_metrics_options` asks for one (:127-190)."""
        from ..common.datatypes import Role
        if placement is None:
            from ..rl.placement import RolePlacement
            placement = RolePlacement(cluster_config.role_to_mesh, make_groups=False)
        r2r = {"rollout": placement.ranks(Role.ROLLOUT), "actor": placement.ranks(Role.ACTOR),
               "refer": placement.ranks(Role.REFERENCE)}
        writer = None
        opts = getattr(cluster_config.training_config, "perf_metrics_options", None)
        if opts is not None and getattr(opts, "enable_trace_writer", False):
            import os
            import tempfile

            from .perfetto import write_spans
            trace_dir = getattr(opts, "log_dir", None) or os.path.join(tempfile.gettempdir(), "tunix_b200_traces")
            count = [0]

            def writer(spans):
                count[0] += 1
                t0 = min((s.begin for s in spans), default=0.0)
                write_spans(spans, os.path.join(trace_dir, f"step_{count[0]:06d}.rank{placement.rank}.json"), t0)
        return PerfMetricsExport.from_role_to_ranks(r2r, writer)

    create_metrics_export_fn = from_cluster_config


def merge_over_ranks(mine: dict, placement=None) -> dict:
    """Every rank contributes its dictionary; step-level times become the max over the controllers, what the serving
    ranks measured appears under `perf/rollout_ranks/...` (max over them). Collective over the job's host group."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return dict(mine)
    box = [None] * dist.get_world_size()
    dist.all_gather_object(box, mine, group=getattr(placement, "host_group", None))
    ctl = set(placement.controllers) if placement is not None else set(range(len(box)))
    out: dict = {}
    for r, d in enumerate(box):
        for k, v in (d or {}).items():
            key = k if r in ctl else k.replace("perf/", "perf/rollout_ranks/", 1)
            out[key] = max(out.get(key, v), v)
    return out


def export_grpo_metrics(tracer: PerfTracer, step_span: Optional[Span] = None, layout: str = COLOCATED) -> dict:
    """Direct form: pick the exporter by layout name."""
    return _EXPORTERS[layout](PerfSpanQuery.of(tracer), step_span)
