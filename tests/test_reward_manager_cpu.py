"""Reward managers: several functions summed, keyword filtering and config injection, shape checks, NaN handling,
worker processes with fallback, the agentic variant; DAPO's overlong reward shaping
(test model: tests/rl/reward_manager_test.py, tests/rl/grpo/dapo_learner_test.py)."""
import os

import numpy as np
import pytest

from tunix_b200.rl import function_registry, reward_manager
from tunix_b200.rl.algorithm_config import DAPOConfig, GRPOConfig


def length_reward(prompts, completions, **kw):
    return [float(len(c)) for c in completions]


def answer_reward(prompts, completions, answer):
    return [1.0 if c.strip() == a else 0.0 for c, a in zip(completions, answer)]


def config_aware(prompts, completions, num_generations):
    return [float(num_generations)] * len(prompts)


def pid_reward(prompts, completions, **kw):
    return [float(os.getpid())] * len(prompts)


def test_sequence_manager_sums_filters_kwargs_and_injects_config():
    cfg = GRPOConfig(num_generations=4)
    rm = function_registry.get_reward_manager("sequence-level")([length_reward, answer_reward, config_aware], cfg)
    out = rm(["p", "q"], ["ab", "7"], answer=["x", "7"], unused_column=[1, 2])
    np.testing.assert_allclose(out["rewards"], [2 + 0 + 4, 1 + 1 + 4])
    assert set(out["per_fn"]) == {"length_reward", "answer_reward", "config_aware"}
    np.testing.assert_allclose(out["per_fn"]["answer_reward"], [0, 1])
    single = reward_manager.SequenceRewardManager(length_reward, cfg)                 # one function, not a list
    np.testing.assert_allclose(single(["p"], ["abc"])["rewards"], [3])
    with pytest.raises(ValueError, match="cannot be empty"):
        reward_manager.SequenceRewardManager([], cfg)


def test_shape_mismatch_is_an_error_and_nan_counts_as_zero():
    cfg = GRPOConfig(num_generations=2)
    bad = reward_manager.SequenceRewardManager([lambda prompts, completions, **kw: [1.0]], cfg)
    with pytest.raises(ValueError, match="returned shape"):
        bad(["a", "b"], ["x", "y"])
    nan = reward_manager.SequenceRewardManager([lambda prompts, completions, **kw: [float("nan"), 2.0], length_reward], cfg)
    out = nan(["a", "b"], ["x", "yy"])
    np.testing.assert_allclose(out["rewards"], [1.0, 4.0])


def test_worker_processes_and_fallback_for_unpicklable_functions():
    cfg = GRPOConfig(num_generations=2, reward_num_workers=2, reward_worker_timeout_seconds=60.0)
    rm = reward_manager.SequenceRewardManager([pid_reward, answer_reward], cfg)
    try:
        out = rm(["a", "b", "c", "d"], ["1", "2", "3", "4"], answer=["1", "x", "3", "x"])
        assert all(int(p) != os.getpid() for p in out["per_fn"]["pid_reward"])       # evaluated in worker processes
        np.testing.assert_allclose(out["per_fn"]["answer_reward"], [1, 0, 1, 0])     # columns were split with the rows
        local = reward_manager.SequenceRewardManager([lambda prompts, completions, **kw: [float(os.getpid())] * len(prompts)], cfg)
        assert all(int(p) == os.getpid() for p in local(["a", "b"], ["x", "y"])["rewards"])   # a lambda cannot travel
        local.close()
    finally:
        rm.close()
    rm.close()                                                                       # closing twice is fine


def test_agentic_manager_adds_environment_rewards():
    cfg = GRPOConfig(num_generations=2)
    rm = function_registry.get_reward_manager("agentic-sequence-level")([length_reward], cfg)
    out = rm(["p", "q"], ["ab", "c"], env_rewards=[0.5, -1.0])
    np.testing.assert_allclose(out["rewards"], [2.5, 0.0])
    np.testing.assert_allclose(out["per_fn"]["env"], [0.5, -1.0])
    np.testing.assert_allclose(rm(["p"], ["abc"])["rewards"], [3.0])


def test_dapo_overlong_buffer_penalises_only_the_tail_of_the_budget():
    from tunix_b200.rl.grpo.grpo_learner import DAPOLearner
    cfg = DAPOConfig(num_generations=2, overlong_buffer={"enable": True, "overlong_buffer_length": 4, "overlong_buffer_penalty": 1.0,
                                                         "max_response_length": 12})
    learner = DAPOLearner.__new__(DAPOLearner)
    learner.algo_config = cfg
    r = np.zeros(5, np.float32)
    shaped = learner._shape_rewards(r, None, [2, 8, 10, 12, 16])
    np.testing.assert_allclose(shaped, [0, 0, -0.5, -1.0, -2.0])                     # free up to 8 tokens, linear afterwards
    cfg.overlong_buffer["enable"] = False
    assert learner._shape_rewards(r, None, [16] * 5) is r
    cfg.overlong_buffer = None
    assert learner._shape_rewards(r, None, [16] * 5) is r
