"""Scenarios above the loss math: a GRPO run that stops and resumes in the middle, several passes over a step's data
with a seeded shuffle, and agentic episodes that time out or are cancelled (test model: the scenarios of
tests/rl/grpo/grpo_learner_test.py and tests/rl/agentic/agentic_grpo_learner_test.py). CPU, tiny models."""
import asyncio
import time

import numpy as np
import pytest
import torch

from tunix_b200.lora import LoraProvider, apply_lora_to_model
from tunix_b200.models.transformer import create_model
from tunix_b200.rl.agentic.agents.agent_types import TrajectoryStatus
from tunix_b200.rl.agentic.agents.model_agent import ModelAgent
from tunix_b200.rl.agentic.environments.task_environment import TaskEnvironment
from tunix_b200.rl.agentic.trajectory.trajectory_collect_engine import TrajectoryCollectEngine
from tunix_b200.rl.algorithm_config import GRPOConfig
from tunix_b200.rl.grpo.grpo_learner import GRPOLearner
from tests.test_rl_learners_cpu import _cfg, _cluster
from tests.test_sampler_cpu import CharTok


def _lora_actor():
    actor = create_model(_cfg(), seed=0)
    apply_lora_to_model(actor, LoraProvider(module_path=r".*(q_proj|v_proj)", rank=4, alpha=8.0))
    return actor


def _lora_state(model):
    return {n: p.detach().clone() for n, p in model.named_parameters() if "lora" in n}


class _Recorder:
    """A reward function that remembers which prompts it scored."""
    __name__ = "recorder"

    def __init__(self):
        self.seen = []

    def __call__(self, prompts, completions, completion_ids=None, completion_lengths=None, **kw):
        self.seen.append(tuple(prompts))
        return [float((ids[:n] % 7 == 0).mean()) if n else 0.0 for ids, n in zip(completion_ids, completion_lengths)]


def test_grpo_run_resumes_mid_dataset_with_restored_weights(tmp_path):
    data = [{"prompts": [f"{chr(97 + 4 * b + i)}x" for i in range(4)]} for b in range(4)]
    first = _Recorder()
    actor = _lora_actor()
    cl = _cluster(actor, steps=2, tmp=str(tmp_path))
    GRPOLearner(cl, [first], GRPOConfig(num_generations=2, beta=0.0)).train(data)
    assert cl.global_steps == 2
    trained_on = {p for batch in first.seen for p in batch}
    assert trained_on == set(data[0]["prompts"]) | set(data[1]["prompts"])
    after_first = _lora_state(actor)
    cl.close()
    # a new process: same checkpoint directory, same dataset, a higher step limit
    second = _Recorder()
    actor2 = _lora_actor()
    cl2 = _cluster(actor2, steps=4, tmp=str(tmp_path))
    assert cl2.global_steps == 2
    restored = _lora_state(actor2)
    assert restored.keys() == after_first.keys() and all(torch.equal(restored[k], after_first[k]) for k in restored)
    GRPOLearner(cl2, [second], GRPOConfig(num_generations=2, beta=0.0)).train(data)
    assert cl2.global_steps == 4
    assert {p for batch in second.seen for p in batch} == set(data[2]["prompts"]) | set(data[3]["prompts"])   # 0 and 1 were skipped
    assert any(not torch.equal(v, after_first[k]) for k, v in _lora_state(actor2).items())
    assert len(cl2.metrics_logger.get_metric_history("", "rewards/score/mean", "train")) == 2
    cl2.close()
    # a third start with nothing left to do trains on nothing
    third = _Recorder()
    cl3 = _cluster(_lora_actor(), steps=4, tmp=str(tmp_path))
    GRPOLearner(cl3, [third], GRPOConfig(num_generations=2, beta=0.0)).train(data)
    assert third.seen == [] and cl3.global_steps == 4
    cl3.close()


@pytest.mark.parametrize("seed", [None, 11])
def test_several_passes_over_a_step_reuse_the_rollouts_and_shuffle_by_seed(seed):
    """mu = 3: every prompt is generated and scored once per step, the trainer sees each micro-batch three times
    (an optimizer step per pass), and later passes come in the seeded order."""
    rec = _Recorder()
    actor = _lora_actor()
    cl = _cluster(actor, steps=2, mini=4, micro=1)
    learner = GRPOLearner(cl, [rec], GRPOConfig(num_generations=2, beta=0.0, num_iterations=3), data_shuffle_seed=seed)
    order = []
    inner = learner._train_on

    def spy(examples):
        def tap():
            for ex in examples:
                order.append(tuple(ex.completion_ids.reshape(-1).tolist()))
                yield ex
        return inner(tap())
    learner._train_on = spy
    data = [{"prompts": ["ab", "cd", "ef", "gh"]} for _ in range(2)]
    learner.train(data)
    assert cl.global_steps == 2 and len(rec.seen) == 2                                   # scored once per step
    per_step = len(order) // 2
    assert per_step == 4 * 3                                                             # 4 micro-batches x 3 passes
    for s in range(2):
        step = order[s * per_step:(s + 1) * per_step]
        first_pass = step[:4]
        assert sorted(step[4:8]) == sorted(first_pass) and sorted(step[8:]) == sorted(first_pass)
        if seed is None:
            assert step[4:8] == first_pass and step[8:] == first_pass
        else:
            idx = list(range(4)); np.random.default_rng(seed + 1).shuffle(idx)
            assert step[4:8] == [first_pass[i] for i in idx]
    assert cl.actor_trainer.train_steps >= 2 * 3
    cl.close()


def _engine(model_call, env=None, **kw):
    return TrajectoryCollectEngine(ModelAgent(), env or TaskEnvironment(task={"question": "q"}), model_call=model_call,
                                   tokenizer=CharTok(), **kw)


def test_episode_budget_cuts_a_slow_model_call():
    cancelled = []

    async def slow(**kw):
        try:
            await asyncio.sleep(30)
        except asyncio.CancelledError:
            cancelled.append(True)
            raise
    t0 = time.monotonic()
    out = asyncio.run(_engine(slow, timeout=0.2, overlong_filter=True).collect("Token"))
    assert time.monotonic() - t0 < 5 and cancelled == [True]
    assert out["status"] == TrajectoryStatus.TIMEOUT and out["masked_out"] and out["conversation_masks"].sum() == 0


def test_environment_step_limit_is_reported_apart_from_the_episode_budget():
    class SlowEnv(TaskEnvironment):
        async def step_async(self, action):
            await asyncio.sleep(30)

    async def answer(**kw):
        return {"text": "hi", "tokens": [5, 6], "logprobs": [-0.1, -0.1]}
    out = asyncio.run(_engine(answer, SlowEnv(task={"question": "q"}), timeout=60, env_step_timeout=0.1).collect("Trajectory"))
    assert out.status == TrajectoryStatus.ENV_TIMEOUT
    out = asyncio.run(_engine(answer, SlowEnv(task={"question": "q"}), timeout=0.2, env_step_timeout=20).collect("Trajectory"))
    assert out.status == TrajectoryStatus.TIMEOUT                       # the episode's budget ran out first
    out = asyncio.run(_engine(answer, SlowEnv(task={"question": "q"}), timeout=0.2).collect("Trajectory"))
    assert out.status == TrajectoryStatus.TIMEOUT


def test_cancelled_episode_is_marked_and_the_cancellation_propagates():
    started = asyncio.Event() if False else None

    async def run():
        gate = asyncio.Event()

        async def hang(**kw):
            gate.set()
            await asyncio.sleep(30)
        eng = _engine(hang, timeout=60)
        task = asyncio.ensure_future(eng.collect("Trajectory"))
        await gate.wait()
        task.cancel()
        with pytest.raises(asyncio.CancelledError):
            await task
        return eng.agent.trajectory.status
    assert asyncio.run(run()) == TrajectoryStatus.CANCELLED


def test_data_queue_bounds_times_out_and_close_releases_blocked_threads():
    import queue, threading, time
    from tunix_b200.rl.queue.data_queue import SimpleDataQueue
    q = SimpleDataQueue(maxsize=2)
    q.put(1); q.put(2)
    assert q.qsize() == 2
    state = {}

    def producer():
        q.put(3)                                   # full: parks until a get or a close
        state["put_returned"] = True
    t = threading.Thread(target=producer); t.start()
    time.sleep(0.05)
    assert "put_returned" not in state
    assert q.get() == 1                            # FIFO, and makes room
    t.join(2); assert state.get("put_returned")
    assert [q.get(), q.get()] == [2, 3]
    t0 = time.monotonic()
    with pytest.raises(queue.Empty):
        q.get(timeout=0.05)
    assert 0.04 <= time.monotonic() - t0 < 1.0
    with pytest.raises(queue.Empty):
        q.get(block=False)

    def consumer():
        try:
            q.get()
        except queue.Empty:
            state["woken"] = True
    c = threading.Thread(target=consumer); c.start()
    time.sleep(0.05)
    q.close()
    c.join(2); assert state.get("woken") and q.closed
    q.put(9)                                       # dropped after close
    assert q.qsize() == 0
