"""Step-organised timelines, asynchronous spans, span post-processing, trace writer and export
(test model: tunix/perf/experimental/{timeline,timeline_utils,trace_writer,export}_test.py)."""
import concurrent.futures
import json
import threading
import time

import numpy as np
import pytest

from tunix_b200.perf.experimental import constants as C
from tunix_b200.perf.experimental import export, timeline, timeline_utils, trace_writer


def _span(i, name, b, e, tags=None):
    s = timeline.Span(name=name, begin=b, id=i, tags=tags)
    s.end = e
    return s


def test_timeline_nesting_commit_and_purge():
    tl = timeline.Timeline("host-1", 10.0)
    outer = tl.start_span("outer", 10.0, tags={C.STEP: 0})
    inner = tl.start_span("inner", 10.5)
    assert inner.parent_id == outer.id and outer.parent_id is None
    tl.stop_span(11.0)
    tl.stop_span(12.0)
    tl.start_span("dangling", 12.5)                 # never stopped: purged at the step boundary
    before = tl.committed_steps
    tl.commit_step()
    assert before == [] and len(tl.committed_steps) == 1          # copy on write
    step = tl.committed_steps[0]
    assert sorted(s.name for s in step.values()) == ["inner", "outer"]
    assert step[outer.id].duration == pytest.approx(2.0)
    assert tl.cur_step == {}
    with pytest.raises(ValueError, match="no more spans"):
        tl.stop_span(13.0)
    tl.start_span("backwards", 20.0)
    with pytest.raises(ValueError, match="before it began"):
        tl.stop_span(19.0)
    assert "Committed Step -0" in repr(tl)


def test_span_tags_are_copied_and_overwrite_warns(caplog):
    tags = {"a": 1}
    s = timeline.Span("x", 0.0, 0, tags=tags)
    s.add_tag("b", 2)
    assert tags == {"a": 1} and s.tags == {"a": 1, "b": 2}
    with caplog.at_level("WARNING"):
        s.add_tag("a", 3)
    assert s.tags["a"] == 3 and "overwriting" in caplog.text
    assert not s.ended


def test_async_timeline_closes_span_when_future_completes():
    tl = timeline.AsyncTimeline("cuda0", time.perf_counter())
    fut = concurrent.futures.Future()
    t0 = time.perf_counter()
    tl.span("rollout", t0, waitlist=[fut], tags={C.GROUP: 3})
    assert tl.cur_step == {}                         # nothing recorded while the work is in flight
    threading.Timer(0.05, fut.set_result, args=(None,)).start()
    tl.wait_pending_spans()
    (s,) = tl.cur_step.values()
    assert s.name == "rollout" and s.ended and s.duration >= 0.04 and s.tags == {C.GROUP: 3}
    tl.span("instant", time.perf_counter())          # empty waitlist: closed at once
    assert len(tl.cur_step) == 2
    tl.commit_step()
    assert len(tl.committed_steps[0]) == 2


def test_async_span_failure_is_logged_not_recorded(caplog):
    tl = timeline.AsyncTimeline("cuda0", 0.0)
    fut = concurrent.futures.Future()
    fut.set_exception(RuntimeError("device lost"))
    with caplog.at_level("ERROR"):
        tl.span("broken", 0.0, waitlist=fut)
        tl.wait_pending_spans()
    assert tl.cur_step == {} and "device lost" in caplog.text


def test_batch_async_timelines_share_one_end_time():
    tls = [timeline.AsyncTimeline(f"cuda{i}", 0.0) for i in range(3)]
    batch = timeline.BatchAsyncTimelines(tls)
    ev = threading.Event()                            # anything with wait() can close a span
    batch.span("peft_train", time.perf_counter(), waitlist={"loss": ev})
    threading.Timer(0.02, ev.set).start()
    batch.wait_pending_spans()
    ends = {next(iter(tl.cur_step.values())).end for tl in tls}
    assert len(ends) == 1


def test_timeline_ids():
    assert timeline_utils.is_host_timeline(timeline_utils.generate_host_timeline_id())
    assert timeline_utils.generate_device_timeline_id(3) == "cuda3"
    assert timeline_utils.generate_device_timeline_id("cuda5") == "cuda5"
    import torch
    assert timeline_utils.generate_device_timeline_id(torch.device("cuda:2")) == "cuda2"
    assert timeline_utils.generate_device_timeline_ids(np.arange(4).reshape(2, 2)) == ["cuda0", "cuda1", "cuda2", "cuda3"]
    q = timeline_utils.generate_queued_timeline_id("cuda1")
    assert timeline_utils.is_queued_timeline(q) and not timeline_utils.is_queued_timeline("cuda1")
    with pytest.raises(ValueError):
        timeline_utils.generate_device_timeline_id(1.5)


def test_only_allowed_span_names():
    tl = timeline.Timeline("cuda0", 0.0)
    assert not timeline_utils.is_timeline_only_of_allowed_type(tl, [C.ROLLOUT])          # empty
    tl.start_span(C.ROLLOUT, 0.0); tl.stop_span(1.0)
    assert not timeline_utils.is_timeline_only_of_allowed_type(tl, [C.ROLLOUT])          # not committed yet
    assert timeline_utils.is_timeline_only_of_allowed_type(tl, [C.ROLLOUT], include_cur_step=True)
    tl.commit_step()
    assert timeline_utils.is_timeline_only_of_allowed_type(tl, [C.ROLLOUT])
    tl.start_span(C.PEFT_TRAIN, 1.0); tl.stop_span(2.0); tl.commit_step()
    assert not timeline_utils.is_timeline_only_of_allowed_type(tl, [C.ROLLOUT])


def test_sequentialize_overlapping_spans():
    spans = {0: _span(0, "a", 0.0, 4.0), 1: _span(1, "b", 1.0, 6.0), 2: _span(2, "c", 2.0, 7.0),
             3: _span(3, "d", 10.0, 11.0), 4: _span(4, "inside", 10.2, 10.8)}
    active, queue = timeline_utils.sequentialize_overlapping_spans(spans)
    assert (active[0].begin, active[0].end) == (0.0, 4.0)
    assert (active[1].begin, active[1].end) == (4.0, 6.0)
    assert (active[2].begin, active[2].end) == (6.0, 7.0)
    assert (active[3].begin, active[3].end) == (10.0, 11.0)
    assert 4 not in active                                      # no active time of its own
    assert (queue[1].begin, queue[1].end, queue[1].tags) == (1.0, 4.0, {C.NAME: "b"})
    assert (queue[2].begin, queue[2].end) == (4.0, 6.0)          # queue spans do not overlap either
    assert queue[4].name == C.QUEUE and (queue[4].begin, queue[4].end) == (10.2, 11.0)
    qs = sorted(queue.values(), key=lambda s: s.begin)
    assert all(a.end <= b.begin for a, b in zip(qs, qs[1:]))


def test_span_names_and_lanes():
    assert trace_writer._create_span_name("x", {}) == "x"
    assert trace_writer._create_span_name(C.PEFT_TRAIN, {C.STEP: 4, C.ROLE: "actor", C.MINI_BATCH: 1, C.MICRO_BATCH: 0}) == \
        "peft_train (step=4, role=actor, mini_batch=1, micro_batch=0)"
    assert trace_writer._create_span_name(C.ROLLOUT, {C.GROUP: 7, C.PAIR: 2}) == "rollout (group_id=7, pair_index=2)"
    assert trace_writer._create_span_name(C.QUEUE, {C.NAME: "rollout"}) == "queue (name=rollout)"
    assert trace_writer._create_span_name(C.REFERENCE_INFERENCE, {C.PAIR: 2}) == "reference_inference"
    lanes, n = trace_writer._assign_lanes([_span(0, "a", 0, 4), _span(1, "b", 1, 2), _span(2, "c", 2, 5), _span(3, "d", 4, 6)])
    assert n == 2 and lanes == {0: 0, 1: 1, 2: 1, 3: 0}
    assert trace_writer._assign_lanes([]) == ({}, 0)


def _two_timelines():
    host = timeline.Timeline("host-1", 100.0)
    host.start_span(C.DATA_LOADING, 100.0, tags={C.STEP: 0}); host.stop_span(100.5); host.commit_step()
    dev = timeline.AsyncTimeline("cuda1", 100.0)
    dev._finish(*dev._reserve(), C.ROLLOUT, 100.1, 101.0, {C.GROUP: 0})
    dev._finish(*dev._reserve(), C.ROLLOUT, 100.2, 100.9, {C.GROUP: 1})       # overlaps: second lane
    dev.commit_step()
    return {"host-1": host, "cuda1": dev}


def test_trace_writer_file(tmp_path):
    w = trace_writer.PerfettoTraceWriter(str(tmp_path), role_to_devices={"rollout": [1], "actor": np.array([[0, 1]])})
    w.write_timelines({})                                          # nothing to write, no file
    assert not list(tmp_path.iterdir())
    w.write_timelines(_two_timelines())
    ev = json.load(open(w.trace_file_path))["traceEvents"]
    procs = {e["args"]["name"]: e["pid"] for e in ev if e["name"] == "process_name"}
    assert set(procs) == {"host", "role rollout", "role actor"}    # cuda1 serves both roles
    threads = [e for e in ev if e["name"] == "thread_name" and e["pid"] == procs["role rollout"]]
    assert [t["args"]["name"] for t in threads] == ["cuda1", "cuda1 +1"]
    slices = [e for e in ev if e["ph"] == "X" and e["pid"] == procs["role rollout"]]
    assert len({s["tid"] for s in slices}) == 2
    first = min(slices, key=lambda s: s["ts"])
    assert first["name"] == "rollout (group_id=0)" and first["ts"] == pytest.approx(0.1e6) and first["dur"] == pytest.approx(0.9e6)
    host = [e for e in ev if e["ph"] == "X" and e["pid"] == procs["host"]]
    assert host[0]["name"] == "data_loading (step=0)" and host[0]["args"] == {C.STEP: "0"}
    trace_writer.NoopTraceWriter().write_timelines(_two_timelines())


def test_export_in_background_and_from_cluster_config(tmp_path):
    class Cfg:
        role_to_mesh = {"actor": np.array([0, 1]), "rollout": [1]}
    with export.PerfMetricsExport.from_cluster_config(Cfg(), trace_dir=str(tmp_path)) as ex:
        assert ex.export_metrics(_two_timelines()) == {}
        path = ex.trace_file_path
    names = {e["args"]["name"] for e in json.load(open(path))["traceEvents"] if e["name"] == "process_name"}
    assert names == {"host", "role actor", "role rollout"}
    ex.export_metrics(_two_timelines())                             # after shutdown: a warning, no error
    off = export.PerfMetricsExport(enable_trace_writer=False)
    assert off.export_metrics(_two_timelines()) == {} and off.trace_file_path is None
    off.shutdown()
    assert export.log_metric_export_fn({}) == {}


def test_export_takes_the_package_mesh(tmp_path):
    from tunix_b200.parallel.mesh import Mesh

    class Cfg:
        role_to_mesh = {"actor": Mesh((2,), ("fsdp",), ranks=[0, 1]), "rollout": Mesh((1,), ("fsdp",), ranks=[2])}
    ex = export.PerfMetricsExport.from_cluster_config(Cfg(), trace_dir=str(tmp_path))
    assert ex._writer._role_to_devices == {"actor": ["cuda0", "cuda1"], "rollout": ["cuda2"]}
    ex.shutdown()


def test_span_trees_queries_clone_and_merge():
    from tunix_b200.perf import span as sp

    def tree(steps):
        root = sp.SpanGroup("root"); root.begin, root.end = 0.0, 100.0
        for (b, e, leaves) in steps:
            g = sp.SpanGroup("global_step", root); g.begin, g.end = b, e
            for (n, lb, le) in leaves:
                s = sp.Span(n, lb); s.end = le; g.inner.append(s)
        return root
    a = tree([(0, 10, [("rollout", 0, 4)]), (10, 20, [("rollout", 10, 13)])])
    b = tree([(0, 10, [("train", 5, 9)]), (20, 30, [("train", 21, 29)])])
    assert a.outer is a and a.find_first_inner_group("global_step").begin == 0 and a.find_last_inner_group("global_step").begin == 10
    assert a.find_last_inner_group("nope") is None and len(a.find_all_inner_groups("global_step")) == 2
    g0 = a.find_first_inner_group("global_step")
    assert g0.find_last_inner_span("rollout").duration == 4 and g0.find_all_inner_spans("train") == [] and g0.duration == 10
    assert [g.begin for g in sp.span_group_batch_query_first([a, b], "global_step")] == [0, 0]
    assert [g.begin for g in sp.span_group_batch_query_last([a, b], "global_step")] == [10, 20]
    assert [g.begin for g in sp.span_group_batch_query_nth([a, b], "global_step", 1)] == [10, 20]
    assert sp.span_group_batch_query_nth([a], "global_step", 5) == [] and len(sp.span_group_batch_query_all([a, b], "global_step")) == 4
    m = sp.merge_span_group_trees(a, b)
    assert [(g.begin, [s.name for s in g.inner]) for g in m.inner] == [(0, ["rollout", "train"]), (10, ["rollout"]), (20, ["train"])]
    assert len(a.inner) == 2 and len(a.inner[0].inner) == 1                          # inputs untouched
    assert all(g.outer is m for g in m.inner)
    assert len(sp.merge_span_group_trees(a, a).inner[0].inner) == 1                  # duplicates collapse
    with pytest.raises(ValueError, match="Overlap detected"):
        sp.merge_span_group_trees(a, tree([(5, 15, [])]))
    with pytest.raises(ValueError, match="Roots are not identical"):
        sp.merge_span_group_trees(a, sp.SpanGroup("other"))
    text = sp.span_group_tostring(a, born=0.0)
    assert text.splitlines()[0].startswith("- root (0.000000") and "    - rollout (10.000000, 13.000000)" in text
    chain = sp.span_group_stack_clone([a, g0])
    assert [c.name for c in chain] == ["root", "global_step"] and chain[1].outer is chain[0] and chain[1].inner == []
    s = sp.Span("open", 1.0)
    assert not s.ended and sp.clone_span_or_group(s).begin == 1.0


def test_span_tree_from_the_tracer():
    from tunix_b200.perf import span as sp
    from tunix_b200.perf.trace import PerfTracer
    tr = PerfTracer()
    for _ in range(2):
        with tr.span_group("global_step"):
            with tr.span("rollout"):
                pass
            with tr.span("train"):
                pass
    root = sp.tree_from_tracer(tr.spans())
    steps = root.find_all_inner_groups("global_step")
    assert len(steps) == 2 and [x.name for x in steps[0].inner] == ["rollout", "train"]
    assert root.begin == steps[0].begin and root.end == steps[1].end and steps[0].end <= steps[1].begin
