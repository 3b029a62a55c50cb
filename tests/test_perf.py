import json
import threading
import time

from tunix_b200.perf import export, perfetto
from tunix_b200.perf.metrics import PerfSpanQuery
from tunix_b200.perf.trace import NoopTracer, PerfTracer


def test_nested_spans_and_queries(tmp_path):
    tr = PerfTracer()
    with tr.span_group("global_step", step=0) as g:
        for mb in range(2):
            with tr.span("rollout", micro=mb):
                time.sleep(0.002)
        with tr.span("actor_train"):
            with tr.span("peft_train_step"):
                time.sleep(0.001)
        with tr.span("weight_sync"):
            pass
    q = PerfSpanQuery.of(tr)
    assert q.name("rollout").count() == 2
    assert q.name("rollout").tag(micro=1).count() == 1
    assert q.within(g).count() == 5
    m = export.export_grpo_metrics(tr, g)
    assert m["perf/sum/rollout_time"] >= 0.004 and m["perf/global_step_time"] >= m["perf/sum/rollout_time"]
    m2 = export.export_grpo_metrics(tr, g, layout="fully_disaggregated")
    assert "perf/rollout_idle_time" in m2 and "perf/sum/actor_gap_time" in m2
    p = perfetto.write_trace(tr, str(tmp_path / "t.json"))
    ev = json.load(open(p))["traceEvents"]
    assert sum(1 for e in ev if e.get("ph") == "X") == 6


def test_threads_have_separate_stacks_and_noop():
    tr = PerfTracer()

    def work():
        with tr.span("worker"):
            time.sleep(0.001)
    with tr.span("main"):
        t = threading.Thread(target=work, name="w0")
        t.start()
        t.join()
    spans = {s.name: s for s in tr.spans()}
    assert spans["worker"].parent is None and spans["worker"].timeline == "w0"
    n = NoopTracer()
    with n.span("x") as s:
        assert s is None
    assert n.spans() == []


def test_tagged_tracer_query_sequence_and_lanes(tmp_path):
    import json
    from tunix_b200.perf.experimental import constants as C
    from tunix_b200.perf.experimental.tracer import TaggedTracer, assign_lanes, sequentialize, write_chrome_trace
    now = [0.0]
    tr = TaggedTracer(clock=lambda: now[0])
    with tr.tags(**{C.STEP: 3}):
        with tr.span("rollout", timeline="engine", **{C.ROLE: C.ROLLOUT}):
            now[0] = 2.0
        with tr.span("update", timeline="trainer", **{C.ROLE: C.ACTOR, C.MICRO_BATCH: 0}):
            now[0] = 3.0
    tr.add("update", "trainer", 2.5, 4.0, **{C.STEP: 3, C.ROLE: C.ACTOR, C.MICRO_BATCH: 1})
    assert len(tr.query(**{C.STEP: 3})) == 3 and tr.total("update", **{C.ROLE: C.ACTOR}) == 2.5
    seq = sequentialize(tr.query(timeline="trainer"))
    assert [(s.begin, s.end) for s in seq] == [(2.0, 3.0), (3.0, 4.5)]
    lanes = assign_lanes(tr.query(timeline="trainer"))
    assert sorted(lanes.values()) == [0, 1]                      # the two overlapping updates sit on different lanes
    write_chrome_trace(tr.query(), str(tmp_path / "t.json"))
    ev = json.load(open(tmp_path / "t.json"))["traceEvents"]
    assert sum(e["ph"] == "X" for e in ev) == 3


def _fake_step(tr, now, layout_gaps):
    """A scripted global step on a tracer with a hand-driven clock: two micro-batches of rollout -> scoring -> update."""
    from tunix_b200.perf.trace import Span
    spans = []

    def add(name, b, e, parent=None):
        s = Span(name, b, e, parent=parent, timeline="main")
        tr._spans.append(s)
        spans.append(s)
        return s
    g = add("global_step", 0.0, 20.0)
    add("rollout", 0.0, 4.0, g)
    add("refer_inference", 4.0, 5.0, g)
    t0 = add("actor_train", 5.0, 8.0, g)
    add("peft_train_step", 5.5, 7.5, t0)
    add("rollout", 4.0, 9.0, g)              # the next micro-batch was generated while the first one trained
    add("refer_inference", 9.5, 10.5, g)     # 1.5 s after the first update ended
    t1 = add("actor_train", 10.5, 14.0, g)
    add("peft_train_step", 11.0, 13.0, t1)
    add("weight_sync", 16.0, 17.0, g)
    return g


def test_three_layout_exporters_and_selection_from_ranks():
    from tunix_b200.perf.export import PerfMetricsExport, layout_of
    tr = PerfTracer()
    g = _fake_step(tr, None, None)
    colo = PerfMetricsExport.from_role_to_ranks({"rollout": [0, 1], "actor": [0, 1], "refer": [0, 1]})
    apart = PerfMetricsExport.from_role_to_ranks({"rollout": [2, 3], "actor": [0, 1], "refer": [0, 1]})
    full = PerfMetricsExport.from_role_to_ranks({"rollout": [2], "actor": [0], "refer": [1]})
    assert (colo.layout, apart.layout, full.layout) == ("colocated", "rollout_disaggregated", "fully_disaggregated")
    with __import__("pytest").raises(ValueError):
        layout_of({"rollout": [0], "actor": [0], "refer": [1]})
    m = colo(tr)                                                    # finds the last global step by itself
    assert m["perf/global_step_time"] == 20.0 and m["perf/weight_sync_time"] == 1.0
    assert m["perf/sum/rollout_time"] == 9.0 and m["perf/mean/actor_train_time"] == 3.25
    assert m["perf/sum/actor_train_step_time"] == 4.0 and "perf/rollout_idle_time" not in m
    m = apart(tr, g)
    assert m["perf/rollout_idle_time"] == 7.0 and m["perf/first_micro_batch_rollout_time"] == 4.0
    assert m["perf/sum/between_micro_batch_gap_time"] == 1.5 and m["perf/mean/between_micro_batch_gap_time"] == 0.75
    m = full(tr, g)
    assert m["perf/sum/refer_gap_time"] == 6.5 and m["perf/sum/actor_gap_time"] == 9.0 and m["perf/rollout_idle_time"] == 7.0


def test_export_from_cluster_config_writes_a_trace_per_step(tmp_path):
    from tunix_b200.common.configs import ClusterConfig, PerfMetricsOptions, RLTrainingConfig
    from tunix_b200.common.datatypes import Role
    from tunix_b200.perf.export import PerfMetricsExport
    from tunix_b200.rl.placement import RolePlacement
    tc = RLTrainingConfig(eval_every_n_steps=1, perf_metrics_options=PerfMetricsOptions(enable_trace_writer=True,
                                                                                       log_dir=str(tmp_path)))
    r2m = {Role.ACTOR: [0, 1], Role.REFERENCE: [0, 1], Role.ROLLOUT: [2, 3]}
    fn = PerfMetricsExport.from_cluster_config(ClusterConfig(role_to_mesh=r2m, training_config=tc),
                                               RolePlacement(r2m, world=4, rank=0, make_groups=False))
    assert fn.layout == "rollout_disaggregated"
    tr = PerfTracer()
    _fake_step(tr, None, None)
    assert fn(tr)["perf/rollout_idle_time"] == 7.0
    ev = json.load(open(tmp_path / "step_000001.rank0.json"))["traceEvents"]
    assert sum(e.get("ph") == "X" for e in ev) == 10
