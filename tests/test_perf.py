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
