"""From the episode objects of the agentic stack to stored trajectories and back
(tunix/experimental/trajectory/converter.py:25-775).

An agent `Step` (`rl.agentic.agents.agent_types.Step`: one model call and the environment's answer to it) becomes two
ATIF steps: a `TunixAgentStep` (the response, the thought as reasoning content, tool calls recognised in the action,
token ids / masks / log-probs, token counts, the routed experts of the call's prefill) and a `TunixEnvStep` (the
observation as text, reward, terminal flag, the tokens the environment added to the context). A task step (source
user) opens the trajectory. `to_agent_trajectory` inverts the conversion for replay and training from a store."""
from __future__ import annotations

import datetime
import json
from typing import Any, List, Optional, Sequence

import numpy as np

from ...rl.agentic.agents import agent_types
from . import trajectory as T
from .action_converter import extract_tool_calls

AGENT_NAME, AGENT_VERSION = "tunix_b200", "1"


def _text(v: Any) -> str:
    if v is None:
        return ""
    if isinstance(v, str):
        return v
    if isinstance(v, (bytes, bytearray)):
        return bytes(v).decode("utf-8", "replace")
    try:
        return json.dumps(T._jsonable(v), default=str)
    except (TypeError, ValueError):
        return str(v)


def _ints(v) -> Optional[np.ndarray]:
    if v is None:
        return None
    a = np.asarray(v)
    return a.astype(np.int64) if a.size else np.zeros(0, np.int64)


def _now() -> str:
    return datetime.datetime.now(datetime.timezone.utc).isoformat()


def create_task_step(task: Any, step_id: int = 0, timestamp: Optional[str] = None) -> T.TunixEnvStep:
    """The opening step: the task as the user's message (a dict task shows its `question` / `prompt` / `instruction`
    when it has one, the whole task stays in `extra`)."""
    msg = task
    if isinstance(task, dict):
        msg = next((task[k] for k in ("question", "prompt", "instruction", "problem") if task.get(k) is not None), task)
    extra = {"task": T._jsonable(task)} if isinstance(task, dict) else None
    return T.TunixEnvStep(step_id=step_id, source=T.Source.USER, message=_text(msg), timestamp=timestamp or _now(), extra=extra)


def create_agent_step(step: agent_types.Step, step_id: int, model_name: Optional[str] = None, prefill_start: Optional[int] = None,
                      prefill_num_context: Optional[int] = None, timestamp: Optional[str] = None) -> T.TunixAgentStep:
    toks = _ints(step.assistant_tokens)
    metrics = None
    if toks is not None:
        metrics = T.Metrics(completion_tokens=int(len(toks)))
    routed = None if step.routed_experts is None else np.asarray(step.routed_experts).astype(np.int64)
    if routed is not None and (prefill_start is None or prefill_num_context is None):
        # without the call's position in the sequence the rows cannot be aligned later: keep the step, drop the routing
        routed = prefill_start = prefill_num_context = None
    if routed is None:
        prefill_start = prefill_num_context = None
    version = step.policy_version
    return T.TunixAgentStep(
        step_id=step_id, source=T.Source.AGENT, message=step.model_response or "", timestamp=timestamp or _now(),
        model_name=model_name, reasoning_content=step.thought or None, tool_calls=extract_tool_calls(step.action),
        metrics=metrics, llm_call_count=1, mc_return=float(step.mc_return), assistant_tokens=toks,
        assistant_masks=_ints(step.assistant_masks), logprobs=None if step.logprobs is None else np.asarray(step.logprobs, np.float32),
        policy_version=None if version is None else int(version), prefill_routed_experts=routed, prefill_start=prefill_start,
        prefill_num_context=prefill_num_context, extra={"info": T._jsonable(step.info)} if step.info else None)


def create_env_step(step: agent_types.Step, step_id: int, source_call_ids: Optional[Sequence[str]] = None,
                    timestamp: Optional[str] = None) -> T.TunixEnvStep:
    """The environment's answer; when the agent step made tool calls the observation is attached as their results."""
    text = _text(step.observation)
    obs = None
    if source_call_ids:
        obs = T.Observation(results=[T.ObservationResult(source_call_id=c, content=text) for c in source_call_ids])
    return T.TunixEnvStep(step_id=step_id, source=T.Source.USER, message=text, timestamp=timestamp or _now(), observation=obs,
                          reward=float(step.reward), done=bool(step.done), env_tokens=_ints(step.env_tokens),
                          env_masks=_ints(step.env_masks))


def to_tunix_steps(steps: Sequence[agent_types.Step], first_step_id: int = 1, model_name: Optional[str] = None,
                   prompt_length: Optional[int] = None) -> List[T.Step]:
    """Agent / environment step pairs for the episode's turns. With `prompt_length` (tokens of the rendered prompt) the
    routed experts of every call are given their position: turn 0 covers the prompt and its own routed tokens; a later
    turn starts where the previous call's routing stopped."""
    out: list = []
    sid = first_step_id
    pos = 0                       # sequence position up to which routing has been recorded
    seq = prompt_length or 0      # sequence position where this turn's assistant tokens begin
    for s in steps:
        start = ctx = None
        if s.routed_experts is not None and prompt_length is not None:
            rows = len(s.routed_experts)
            start, ctx = pos, max(min(seq - pos, rows), 0)
            pos += rows
        agent = create_agent_step(s, sid, model_name, start, ctx)
        out.append(agent)
        out.append(create_env_step(s, sid + 1, [c.tool_call_id for c in agent.tool_calls] if agent.tool_calls else None))
        sid += 2
        seq += (0 if s.assistant_tokens is None else len(s.assistant_tokens)) + (0 if s.env_tokens is None else len(s.env_tokens))
    return out


def create_trajectory_metadata(trajectory_id: str, *, prompt_id: Optional[str] = None, group_index: int = 0, session_id: Optional[str] = None,
                               model_name: Optional[str] = None, tool_definitions: Optional[list] = None,
                               hyperparams: Optional[dict] = None, notes: Optional[str] = None) -> T.TunixTrajectoryMetadata:
    return T.TunixTrajectoryMetadata(agent=T.Agent(name=AGENT_NAME, version=AGENT_VERSION, model_name=model_name,
                                                   tool_definitions=tool_definitions), trajectory_id=trajectory_id,
                                     session_id=session_id, notes=notes, prompt_id=prompt_id, group_index=group_index,
                                     status=agent_types.TrajectoryStatus.RUNNING.name, hyperparams=hyperparams)


def update_trajectory_metadata(metadata: T.TunixTrajectoryMetadata, traj: agent_types.Trajectory,
                               steps: Optional[Sequence[T.Step]] = None) -> T.TunixTrajectoryMetadata:
    """The metadata after (part of) the episode: status, reward, the overlong flag, environment timings, the policy
    versions seen, and token totals when the steps are given."""
    status = traj.status.name if isinstance(traj.status, agent_types.TrajectoryStatus) else (str(traj.status) if traj.status else None)
    versions = sorted({int(s.policy_version) for s in traj.steps if s.policy_version is not None})
    metadata.status, metadata.total_reward, metadata.masked_out = status, float(traj.reward), traj.masked_out
    metadata.env_time = T._jsonable(traj.env_time) if traj.env_time else None
    metadata.target_policy_versions = versions or None
    if steps is not None:
        done = [s.metrics.completion_tokens for s in steps if isinstance(s, T.TunixAgentStep) and s.metrics is not None
                and s.metrics.completion_tokens is not None]
        metadata.final_metrics = T.FinalMetrics(total_completion_tokens=int(sum(done)) if done else None, total_steps=len(steps))
    return metadata


def to_tunix_trajectory(traj: agent_types.Trajectory, trajectory_id: str, *, prompt_id: Optional[str] = None, group_index: int = 0,
                        session_id: Optional[str] = None, model_name: Optional[str] = None, prompt_length: Optional[int] = None,
                        hyperparams: Optional[dict] = None) -> T.TunixTrajectory:
    steps: list = [create_task_step(traj.task, 0)] + to_tunix_steps(traj.steps, 1, model_name, prompt_length)
    meta = create_trajectory_metadata(trajectory_id, prompt_id=prompt_id, group_index=group_index, session_id=session_id,
                                      model_name=model_name, hyperparams=hyperparams)
    update_trajectory_metadata(meta, traj, steps)
    return meta.create_trajectory(steps)


def log_trajectory(store, traj: T.TunixTrajectory) -> None:
    """Write a whole trajectory through the step-level interface of a store."""
    meta = traj.metadata()
    if not traj.steps:
        store.update_metadata(meta)
    for s in traj.steps:
        store.add_step(s, meta)


def to_agent_trajectory(traj: T.TunixTrajectory) -> agent_types.Trajectory:
    """The episode object back from a stored trajectory: every agent step with the environment step that follows it."""
    out = agent_types.Trajectory()
    steps = list(traj.steps)
    if steps and not isinstance(steps[0], T.TunixAgentStep):
        task = (steps[0].extra or {}).get("task")
        out.task = task if task is not None else steps[0].message
        steps = steps[1:]
    i = 0
    while i < len(steps):
        a = steps[i]
        if not isinstance(a, T.TunixAgentStep):
            i += 1
            continue
        e = steps[i + 1] if i + 1 < len(steps) and isinstance(steps[i + 1], T.TunixEnvStep) else None
        act = None
        if a.tool_calls:
            act = agent_types.Action(action=[{"id": c.tool_call_id, "type": "function",
                                              "function": {"name": c.function_name, "arguments": dict(c.arguments)}} for c in a.tool_calls])
        out.steps.append(agent_types.Step(
            thought=a.reasoning_content or "", action=act, observation=None if e is None else e.message, model_response=a.message,
            info=dict((a.extra or {}).get("info") or {}), reward=0.0 if e is None or e.reward is None else float(e.reward),
            done=bool(e.done) if e is not None and e.done is not None else False, mc_return=float(a.mc_return or 0.0),
            assistant_tokens=a.assistant_tokens, assistant_masks=a.assistant_masks, logprobs=a.logprobs,
            env_tokens=None if e is None else e.env_tokens, env_masks=None if e is None else e.env_masks,
            policy_version=a.policy_version, routed_experts=a.prefill_routed_experts))
        i += 2 if e is not None else 1
    out.step_idx = len(out.steps) - 1
    out.reward = float(traj.total_reward or 0.0)
    out.masked_out = traj.masked_out
    out.env_time = dict(traj.env_time or {})
    if traj.status:
        out.status = getattr(agent_types.TrajectoryStatus, traj.status, agent_types.TrajectoryStatus.RUNNING)
    return out
