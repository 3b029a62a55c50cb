"""ATIF trajectories: schema rules, extension packing and class resolution, tool-call extraction, the step-level
stores with their writer thread, conversion from and to agent episodes
(test model: tunix/experimental/trajectory/{trajectory,action_converter,converter,*_store,async_writer}_test.py)."""
import json
import threading
import time

import numpy as np
import pytest

from tunix_b200.experimental.trajectory import action_converter, async_writer, base_store, converter, db_engine
from tunix_b200.experimental.trajectory import trajectory as T
from tunix_b200.experimental.trajectory.file_store import FileTrajectoryStore
from tunix_b200.experimental.trajectory.in_memory_store import InMemoryTrajectoryStore
from tunix_b200.experimental.trajectory.sql_store import SqlTrajectoryStore
from tunix_b200.rl.agentic.agents import agent_types


def _traj(tid="t1", prompt_id="p0", group_index=1, reward=1.0):
    steps = [T.TunixEnvStep(step_id=0, source="user", message="2+2?", env_tokens=[1, 2, 3], env_masks=[0, 0, 0]),
             T.TunixAgentStep(step_id=1, source="agent", message="4", reasoning_content="add", assistant_tokens=np.array([7, 8]),
                              assistant_masks=[1, 1], logprobs=[-0.5, -0.25], policy_version=3, mc_return=1.0, llm_call_count=1,
                              tool_calls=[T.ToolCall(tool_call_id="c1", function_name="calc", arguments={"e": "2+2"})],
                              metrics=T.Metrics(prompt_tokens=3, completion_tokens=2),
                              prefill_routed_experts=np.arange(5 * 2 * 2).reshape(5, 2, 2), prefill_start=0, prefill_num_context=3),
             T.TunixEnvStep(step_id=2, source="user", message="ok", reward=reward, done=True)]
    return T.TunixTrajectory(agent=T.Agent(name="a", version="1", model_name="tiny"), trajectory_id=tid, session_id="run", prompt_id=prompt_id,
                             group_index=group_index, status="SUCCEEDED", total_reward=reward, steps=steps, extra={"mine": 1})


def test_schema_rules():
    with pytest.raises(ValueError, match="only applicable when source is 'agent'"):
        T.Step(step_id=1, source="user", message="x", model_name="m")
    with pytest.raises(ValueError, match="must be absent when llm_call_count is 0"):
        T.Step(step_id=1, source="agent", message="x", llm_call_count=0, reasoning_content="r")
    T.Step(step_id=1, source="agent", message="dispatch", llm_call_count=0, tool_calls=[T.ToolCall(tool_call_id="c", function_name="f")])
    with pytest.raises(ValueError, match="unknown field"):
        T.Step.from_json({"step_id": 1, "source": "user", "message": "x", "mesage": "typo"})
    with pytest.raises(ValueError, match="either trajectory_id or trajectory_path"):
        T.SubagentTrajectoryRef(session_id="s")
    with pytest.raises(ValueError):
        T.ToolCall(tool_call_id="", function_name="f")
    with pytest.raises(ValueError, match="only applicable when source is 'agent'"):
        T.TunixAgentStep(step_id=0, source="user", message="x")
    with pytest.raises(ValueError, match="'system' or 'user'"):
        T.TunixEnvStep(step_id=0, source="agent", message="x")
    with pytest.raises(ValueError, match="all None or all set"):
        T.TunixAgentStep(step_id=0, source="agent", message="x", prefill_start=0)
    with pytest.raises(ValueError, match="prefill_num_context must be in"):
        T.TunixAgentStep(step_id=0, source="agent", message="x", prefill_routed_experts=np.zeros((2, 1, 1), int), prefill_start=0,
                         prefill_num_context=3)
    with pytest.raises(ValueError, match="integer array"):
        T.TunixAgentStep(step_id=0, source="agent", message="x", assistant_tokens=[[1, 2]])
    with pytest.raises(ValueError, match="consecutive"):
        T.Trajectory(agent=T.Agent(name="a", version="1"), steps=[T.Step(step_id=2, source="user", message="x")])
    with pytest.raises(TypeError, match="EXTENSIONS_KEY"):
        import dataclasses

        @dataclasses.dataclass
        class NoKey(T.Step):
            mine: int = 0


def test_extensions_pack_into_plain_atif_and_come_back_exactly():
    tr = _traj()
    atif = tr.to_atif_trajectory()
    assert type(atif) is T.Trajectory and [s.step_id for s in atif.steps] == [1, 2, 3] and all(type(s) is T.Step for s in atif.steps)
    assert atif.extra["mine"] == 1 and atif.extra[T.TUNIX_EXTENSIONS_KEY]["prompt_id"] == "p0"
    packed = atif.steps[1].extra[T.TUNIX_EXTENSIONS_KEY]
    assert packed["assistant_tokens"] == [7, 8] and packed["prefill_start"] == 0 and np.shape(packed["prefill_routed_experts"]) == (5, 2, 2)
    doc = json.loads(json.dumps(atif.to_json()))                       # what a foreign ATIF reader gets
    assert doc["schema_version"] == "ATIF-v1.7" and doc["steps"][1]["tool_calls"][0]["function_name"] == "calc"
    back = T.TunixTrajectory.from_json(doc)
    assert isinstance(back.steps[1], T.TunixAgentStep) and isinstance(back.steps[2], T.TunixEnvStep)
    assert [s.step_id for s in back.steps] == [0, 1, 2] and back.extra == {"mine": 1} and back.steps[1].extra is None
    np.testing.assert_array_equal(back.steps[1].assistant_tokens, [7, 8])
    np.testing.assert_array_equal(back.steps[1].prefill_routed_experts, tr.steps[1].prefill_routed_experts)
    np.testing.assert_allclose(back.steps[1].logprobs, [-0.5, -0.25])
    assert (back.prompt_id, back.group_index, back.total_reward, back.steps[2].done) == ("p0", 1, 1.0, True)
    own = T.TunixTrajectory.from_json(json.loads(json.dumps(tr.to_json())))             # the class's own JSON reads too
    assert own.steps[1].policy_version == 3 and own.to_json() == back.to_json()
    fm = back.compute_final_metrics()
    assert (fm.total_prompt_tokens, fm.total_completion_tokens, fm.total_steps) == (3, 2, 3)


def test_metadata_class_is_resolved_from_the_packed_keys():
    import dataclasses
    base = _traj().to_atif_trajectory().metadata()
    assert T.TrajectoryMetadata.resolve_subclass(base) is T.TunixTrajectoryMetadata
    plain = T.TrajectoryMetadata(agent=T.Agent(name="a", version="1"), trajectory_id="x")
    assert T.TrajectoryMetadata.resolve_subclass(plain) is T.TrajectoryMetadata and plain.get_extensions() == {}
    assert base.get_extensions()["status"] == "SUCCEEDED"
    # a document written by a newer writer with a key this class does not know: the class still resolves, the key stays
    doc = base.to_json()
    doc["extra"][T.TUNIX_EXTENSIONS_KEY] = {**{k: None for k in ()}, **doc["extra"][T.TUNIX_EXTENSIONS_KEY], "from_the_future": 1,
                                            **{f: doc["extra"][T.TUNIX_EXTENSIONS_KEY].get(f, 0) for f in
                                               ("prompt_id", "group_index", "target_policy_versions", "status", "total_reward", "masked_out",
                                                "hyperparams", "env_time", "reward_time")}}
    newer = T.TrajectoryMetadata.from_json(doc)
    assert T.TrajectoryMetadata.resolve_subclass(newer) is T.TunixTrajectoryMetadata
    got = T.TunixTrajectoryMetadata.from_atif_metadata(newer)
    assert got.prompt_id == "p0" and got.extra[T.TUNIX_EXTENSIONS_KEY] == {"from_the_future": 1}

    @dataclasses.dataclass
    class Narrow(T.TrajectoryMetadata):
        EXTENSIONS_KEY = "_narrow"
        colour: str = "red"
    try:
        n = Narrow(agent=T.Agent(name="a", version="1"), trajectory_id="n", colour="blue").to_atif_metadata()
        assert n.extra == {"_narrow": {"colour": "blue"}} and T.TrajectoryMetadata.resolve_subclass(n) is Narrow
        assert Narrow.from_atif_metadata(n).colour == "blue"
    finally:
        T.TrajectoryMetadata._SUBCLASSES.remove(Narrow)


def test_tool_calls_from_every_shape_of_action():
    x = action_converter.extract_tool_calls
    assert x(None) is None and x(3) is None and x(np.zeros(2)) is None and x("") is None and x("just text") is None and x({}) is None
    openai = x(agent_types.Action(action=[{"id": "a", "type": "function", "function": {"name": "calc", "arguments": '{"e": "1+1"}'}}]))
    assert (openai[0].tool_call_id, openai[0].function_name, openai[0].arguments) == ("a", "calc", {"e": "1+1"})
    anth = x({"type": "tool_use", "id": "t", "name": "n", "input": {"k": 1}})
    assert (anth[0].tool_call_id, anth[0].function_name, anth[0].arguments) == ("t", "n", {"k": 1})
    assert x({"tool": "search", "q": "x", "n": 2})[0].arguments == {"q": "x", "n": 2}
    assert (x({"move": "left"})[0].function_name, x({"move": "left"})[0].arguments) == ("action", {"move": "left"})
    assert x({"id": "only"}) is None
    fenced = x('```json\n{"name": "t", "args": {"z": 2}}\n```')
    assert (fenced[0].function_name, fenced[0].arguments) == ("t", {"z": 2})
    hermes = x('pre <tool_call>{"name": "search", "arguments": {"q": "x"}}</tool_call> mid '
               '<tool_call><name>f</name><arguments>{"a": 1}</arguments></tool_call>')
    assert [(c.tool_call_id, c.function_name, c.arguments) for c in hermes] == [("call_1", "search", {"q": "x"}), ("call_2", "f", {"a": 1})]
    swe = x("<function=bash>\n<parameter=command>ls -l</parameter>\n<parameter=timeout>5</parameter>\n</function>")
    assert swe[0].function_name == "bash" and swe[0].arguments == {"command": "ls -l", "timeout": "5"}
    assert x('<invoke name="get"><parameter name="url">http://x</parameter></invoke>')[0].arguments == {"url": "http://x"}
    assert x("<function=note>free text</function>")[0].arguments == {"input": "free text"}
    assert x('<function=j>{"a": 1}</function>')[0].arguments == {"a": 1}
    mixed = x([{"name": "a"}, '<tool_call>{"name": "b"}</tool_call>', 5, T.ToolCall(tool_call_id="k", function_name="c")])
    assert [c.function_name for c in mixed] == ["a", "b", "c"] and mixed[0].tool_call_id == "call_1"

    class Obj:
        def __init__(self):
            self.name, self.arguments = "o", {"p": 1}
    assert x(Obj())[0].arguments == {"p": 1}
    assert x({"name": "bad", "arguments": "not json"})[0].arguments == {}


def _episode():
    ep = agent_types.Trajectory(task={"question": "What is 2+2?", "answer": "4"})
    call = {"name": "calculator", "arguments": {"expression": "2+2"}}
    ep.steps = [
        agent_types.Step(thought="use the tool", action=agent_types.Action(action=[call]), observation={"calculator": "4"},
                         model_response="<tool_call>...</tool_call>", reward=0.0, done=False, mc_return=1.0,
                         assistant_tokens=np.array([5, 6, 7]), assistant_masks=np.ones(3, np.int32), logprobs=np.array([-.1, -.2, -.3], np.float32),
                         env_tokens=np.array([9, 9]), env_masks=np.zeros(2, np.int32), policy_version=2,
                         routed_experts=np.zeros((6, 1, 2), np.int16), info={"k": 1}),
        agent_types.Step(thought="", action=agent_types.Action(action="4"), observation=None, model_response="4", reward=1.0, done=True,
                         mc_return=1.0, assistant_tokens=np.array([8]), assistant_masks=np.ones(1, np.int32),
                         logprobs=np.array([-.4], np.float32), policy_version=3, routed_experts=np.zeros((6, 1, 2), np.int16))]
    ep.reward, ep.status, ep.masked_out, ep.env_time = 1.0, agent_types.TrajectoryStatus.SUCCEEDED, False, {"reset_latency": 0.01}
    return ep


def test_episode_to_trajectory_and_back():
    ep = _episode()
    tr = converter.to_tunix_trajectory(ep, "traj-7", prompt_id="p7", group_index=2, model_name="tiny", prompt_length=4)
    assert [type(s).__name__ for s in tr.steps] == ["TunixEnvStep", "TunixAgentStep", "TunixEnvStep", "TunixAgentStep", "TunixEnvStep"]
    assert tr.steps[0].message == "What is 2+2?" and tr.steps[0].extra["task"]["answer"] == "4"
    a0, e0, a1 = tr.steps[1], tr.steps[2], tr.steps[3]
    assert a0.tool_calls[0].function_name == "calculator" and a0.reasoning_content == "use the tool" and a0.metrics.completion_tokens == 3
    assert e0.observation.results[0].source_call_id == a0.tool_calls[0].tool_call_id and json.loads(e0.message) == {"calculator": "4"}
    assert (a0.prefill_start, a0.prefill_num_context) == (0, 4)                  # turn 0: the prompt is the context
    assert (a1.prefill_start, a1.prefill_num_context) == (6, 3)                  # rows 6..: 1 unrouted tail + 2 env tokens before turn 1
    assert a1.tool_calls is None and tr.steps[4].done and tr.steps[4].reward == 1.0
    assert (tr.status, tr.total_reward, tr.target_policy_versions, tr.final_metrics.total_completion_tokens) == ("SUCCEEDED", 1.0, [2, 3], 4)
    no_pos = converter.to_tunix_trajectory(ep, "t", prompt_length=None)
    assert no_pos.steps[1].prefill_routed_experts is None                         # routing without positions is not stored
    back = converter.to_agent_trajectory(T.TunixTrajectory.from_json(json.loads(json.dumps(tr.to_atif_trajectory().to_json()))))
    assert back.task["answer"] == "4" and len(back.steps) == 2 and back.status == agent_types.TrajectoryStatus.SUCCEEDED
    np.testing.assert_array_equal(back.steps[0].assistant_tokens, [5, 6, 7]); np.testing.assert_array_equal(back.steps[0].env_tokens, [9, 9])
    assert back.steps[0].policy_version == 2 and back.steps[1].done and back.steps[1].reward == 1.0 and back.steps[0].info == {"k": 1}
    assert action_converter.extract_tool_calls(back.steps[0].action)[0].arguments == {"expression": "2+2"}


@pytest.mark.parametrize("kind", ["memory", "file", "sql", "sql-memory"])
def test_stores_share_one_behaviour(kind, tmp_path):
    make = {"memory": InMemoryTrajectoryStore, "file": lambda: FileTrajectoryStore(str(tmp_path / "root")),
            "sql": lambda: SqlTrajectoryStore(f"sqlite:///{tmp_path}/t.db"), "sql-memory": lambda: SqlTrajectoryStore("sqlite://")}[kind]
    st = make()
    assert isinstance(st, base_store.TrajectoryReader) and isinstance(st, base_store.TrajectoryWriter)
    a, b = _traj("run/a.1", "p0", 0, 1.0), _traj("b", "p1", 1, 0.0)
    meta = a.metadata()
    meta.status = "RUNNING"
    st.add_step(a.steps[0], meta)
    a.steps[0].message = "changed after the call"                  # the store took a snapshot
    st.add_step(a.steps[1], meta)
    st.flush()
    got = st.get_trajectories(["run/a.1"])[0]
    assert isinstance(got, T.TunixTrajectory) and len(got.steps) == 2 and got.status == "RUNNING" and got.steps[0].message == "2+2?"
    st.add_step(a.steps[2], a.metadata())
    converter.log_trajectory(st, b)
    st.update_metadata(T.TunixTrajectoryMetadata(agent=T.Agent(name="a", version="1"), trajectory_id="empty", prompt_id="p2"))
    st.flush()
    metas = st.get_trajectories_metadata()
    assert sorted(m.trajectory_id for m in metas) == ["b", "empty", "run/a.1"] and all(isinstance(m, T.TunixTrajectoryMetadata) for m in metas)
    assert [m.prompt_id for m in st.get_trajectories_metadata(["empty", "b"])] == ["p2", "p1"]
    full = st.get_trajectories(["b", "run/a.1", "empty"])
    assert [len(t.steps) for t in full] == [3, 3, 0] and full[1].status == "SUCCEEDED"
    np.testing.assert_array_equal(full[0].steps[1].assistant_tokens, [7, 8])
    with pytest.raises(base_store.TrajectoryNotFoundError):
        st.get_trajectories(["nope"])
    with pytest.raises(base_store.TrajectoryMetadataNotFoundError):
        st.get_trajectories_metadata(["nope"])
    with pytest.raises(ValueError, match="trajectory_id must be set"):
        st.update_metadata(T.TrajectoryMetadata(agent=T.Agent(name="a", version="1")))
    cfg = st.to_config()
    st.close(); st.close()
    if kind in ("file", "sql"):                                    # a second process opens the same data from the config
        again = base_store.TrajectoryStore.from_config(json.loads(json.dumps(cfg)))
        assert type(again) is type(st) and len(again.get_trajectories(["run/a.1"])[0].steps) == 3
        with pytest.raises(ValueError, match="not a"):
            InMemoryTrajectoryStore.from_config(cfg)
        again.close()
    assert base_store.TrajectoryStore.from_config(None) is None
    with pytest.raises(ValueError, match="unknown trajectory store type"):
        base_store.TrajectoryStore.from_config({"store_type": "tape"})


def test_sql_queries_and_url_handling(tmp_path):
    st = SqlTrajectoryStore(f"sqlite:///{tmp_path}/q.db")
    for i, (pid, status, r) in enumerate([("p0", "SUCCEEDED", 1.0), ("p0", "FAILED", 0.0), ("p1", "SUCCEEDED", 0.5)]):
        t = _traj(f"t{i}", pid, i, r)
        t.status = status
        converter.log_trajectory(st, t)
    st.flush()
    assert st.find_trajectory_ids(prompt_id="p0") == ["t0", "t1"] and st.find_trajectory_ids(status="SUCCEEDED", min_total_reward=0.75) == ["t0"]
    assert st.find_trajectory_ids(limit=2) == ["t0", "t1"] and st.count_steps("t2") == 3 and st.write_errors == 0
    other = SqlTrajectoryStore(f"sqlite:///{tmp_path}/q.db")           # the same file: one shared connection
    assert other._h.engine is st._h.engine
    st.close()
    assert other.count_steps("t0") == 3                                 # still open for the other holder
    other.close()
    assert db_engine.redact_url("postgresql://user:secret@host/db") == "postgresql://user:***@host/db"
    assert db_engine.EngineConfig("sqlite:////abs/x.db").path() == "/abs/x.db" and db_engine.EngineConfig("sqlite:///rel/x.db").path() == "rel/x.db"
    assert db_engine.EngineConfig("sqlite://").in_memory and db_engine.EngineConfig("plain/file.db").path() == "plain/file.db"
    with pytest.raises(ValueError, match="only sqlite"):
        db_engine.EngineConfig("postgresql://u:p@h/db").path()
    assert SqlTrajectoryStore("sqlite://").to_redacted_config()["url"] == "sqlite://"


def test_async_writer_backpressure_errors_flush_and_close():
    gate, seen = threading.Event(), []

    class W(async_writer.AsyncWriter):
        def _process_task(self, task):
            gate.wait(5)
            if task == "bad":
                raise IOError("disk full")
            seen.append(task)
    w = W("w", max_queue_size=2)
    w._enqueue(1); w._enqueue("bad"); w._enqueue(3)                    # one in the worker's hands, two queued
    import queue
    with pytest.raises(queue.Full):
        w._enqueue(4, timeout=0.05)                                    # producers wait when the queue is full
    gate.set()
    assert w.flush(5) and seen == [1, 3] and w.errors == 1 and w.written == 2
    w.close(); w.close()
    assert w.is_closed
    with pytest.raises(async_writer.WriterClosedError):
        w._enqueue(5)
    with pytest.raises(ValueError):
        W("w", max_queue_size=0)


def test_explorer_reads_atif_stores(tmp_path):
    import io
    from tunix_b200.experimental.trajectory import explorer
    root = str(tmp_path / "atif")
    with FileTrajectoryStore(root) as st:
        for i, r in enumerate([1.0, 0.25]):
            converter.log_trajectory(st, converter.to_tunix_trajectory(_episode(), f"traj-{i}", prompt_id="p", group_index=i))
        st.flush()
    out = io.StringIO()
    assert explorer.main([root, "list"], out=out) == 0
    lines = out.getvalue().strip().splitlines()
    assert len(lines) == 2 and "group=p" in lines[0] and "steps=2" in lines[0] and "reward=1.000" in lines[0]
    out = io.StringIO()
    assert explorer.main([root, "show", "traj-1"], out=out) == 0 and "observation:" in out.getvalue()
    dest = str(tmp_path / "sft.jsonl")
    assert explorer.main([root, "export-sft", dest, "--min-reward", "0.5", "--best-of-group"], out=io.StringIO()) == 0
    rows = [json.loads(x) for x in open(dest)]
    assert len(rows) == 1 and rows[0]["messages"][0] == {"role": "user", "content": "What is 2+2?"} and rows[0]["messages"][-1]["content"] == "4"
    db = f"sqlite:///{tmp_path}/a.db"
    with SqlTrajectoryStore(db) as st:
        converter.log_trajectory(st, converter.to_tunix_trajectory(_episode(), "sql-traj", prompt_id="q"))
        st.flush()
    out = io.StringIO()
    assert explorer.main([f"atif:{db}", "stats"], out=out) == 0 and out.getvalue().count("\n") == 2


def test_async_writer_batches_waiting_tasks_and_isolates_a_failing_one():
    gate, batches, singles = threading.Event(), [], []

    class B(async_writer.AsyncWriter):
        def _process_batch(self, tasks):
            batches.append(list(tasks))
            if "bad" in tasks:
                raise IOError("one row is broken")

        def _process_task(self, task):
            gate.wait(5)
            if task == "bad":
                raise IOError("broken")
            singles.append(task)
    w = B("b", max_queue_size=16, max_batch=8)
    w._enqueue("first")                                    # alone in the worker's hands while the others queue up
    time.sleep(0.05)
    for t in ("a", "bad", "c"):
        w._enqueue(t)
    gate.set()
    assert w.flush(5)
    assert singles[0] == "first" and ["a", "bad", "c"] in batches            # the waiting ones went in as one batch ...
    assert singles[1:] == ["a", "c"] and w.errors == 1 and w.written == 3   # ... and singly after it failed
    w.close()


def test_file_store_rewrites_metadata_only_when_it_changes(tmp_path):
    import os
    st = FileTrajectoryStore(str(tmp_path / "r"))
    tr = _traj("same")
    meta = tr.metadata()
    st.add_step(tr.steps[0], meta); st.flush()
    path = st.get_trajectory_metadata_path("same")
    first = os.stat(path).st_mtime_ns
    time.sleep(0.01)
    st.add_step(tr.steps[1], meta); st.flush()
    assert os.stat(path).st_mtime_ns == first                               # unchanged document: not written again
    meta.status = "FAILED"
    st.add_step(tr.steps[2], meta); st.flush()
    assert os.stat(path).st_mtime_ns != first and st.get_trajectories_metadata(["same"])[0].status == "FAILED"
    st.close()
