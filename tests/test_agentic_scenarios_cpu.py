"""The agentic learner above a single happy run: resume in the middle of a dataset, several passes per batch, running
ahead of the trainer, stale groups, groups without learning signal, eval cadence
(test model: the scenarios of tests/rl/agentic/agentic_grpo_learner_test.py). CPU, tiny models."""
import numpy as np
import pytest
import torch

from tunix_b200 import optim
from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model
from tunix_b200.rl.agentic.agentic_grpo_learner import AgenticGRPOLearner
from tunix_b200.rl.agentic.parser.chat_template_parser import get_parser
from tunix_b200.rl.algorithm_config import GRPOConfig
from tunix_b200.rl.rl_cluster import RLCluster
from tests.test_sampler_cpu import CharTok


def _cluster(steps, tmp=None, eval_every=1000, mini=2):
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16,
                                           num_kv_heads=1)
    actor = create_model(cfg, seed=0)
    tc = RLTrainingConfig(eval_every_n_steps=eval_every, max_steps=steps, actor_optimizer=optim.AdamW(1e-3), mini_batch_size=mini,
                          train_micro_batch_size=mini, checkpoint_root_directory=tmp)
    rc = RolloutConfig(max_tokens_to_generate=5, max_prompt_length=16, temperature=1.0, seed=1, kv_cache_size=64, eos_tokens=[63])
    return actor, RLCluster(actor=actor, tokenizer=CharTok(), cluster_config=ClusterConfig(role_to_mesh={}, training_config=tc,
                                                                                          rollout_config=rc))


class _Scorer:
    __name__ = "scorer"

    def __init__(self, fn=None):
        self.calls, self.fn = 0, fn

    def __call__(self, prompts, completions, completion_lengths=None, completion_ids=None, **kw):
        self.calls += 1
        if self.fn is not None:
            return self.fn(completion_ids, completion_lengths)
        return [float(ids[:n].sum() % 5) for ids, n in zip(completion_ids, completion_lengths)]


def _client(log):
    """A scripted engine: answers depend on how many calls came before, so groups differ."""
    async def call(chat_completions=None, prompt_token_ids=None, max_tokens=None):
        log.append(list(prompt_token_ids))
        n = 2 + len(log) % 3
        return {"text": "x" * n, "tokens": [5 + (3 * len(log) + k) % 50 for k in range(n)], "logprobs": [-1.0] * n}
    return call


def _data(n):
    return [{"prompts": [f"{chr(97 + 2 * b)}{chr(98 + 2 * b)}", f"{chr(65 + 2 * b)}{chr(66 + 2 * b)}"]} for b in range(n)]


def _learner(cl, scorer, log, **kw):
    return AgenticGRPOLearner(cl, [scorer], GRPOConfig(num_generations=2, beta=0.0, **kw.pop("algo", {})), max_concurrency=4,
                              chat_parser=get_parser("raw"), model_client=_client(log), **kw)


def test_resume_in_the_middle_of_the_dataset(tmp_path):
    data = _data(4)
    log1, s1 = [], _Scorer()
    actor, cl = _cluster(2, tmp=str(tmp_path))
    _learner(cl, s1, log1).train(data)
    assert cl.global_steps == 2 and len(log1) == 2 * 2 * 2                       # 2 batches x 2 prompts x 2 generations
    weights = torch.cat([p.detach().reshape(-1).clone() for p in actor.parameters()])
    log2, s2 = [], _Scorer()
    actor2, cl2 = _cluster(4, tmp=str(tmp_path))
    assert cl2.global_steps == 2
    assert torch.equal(torch.cat([p.detach().reshape(-1) for p in actor2.parameters()]), weights)
    learner = _learner(cl2, s2, log2)
    assert learner.policy_version == 2                                           # versions go on from the restored step
    learner.train(data)
    assert cl2.global_steps == 4 and learner.policy_version == 4 and len(log2) == 8
    tok = CharTok()
    seen_first, seen_second = {tuple(p) for p in log1}, {tuple(p) for p in log2}
    assert seen_first.isdisjoint(seen_second)                                    # the resumed run asked about new prompts only
    want = {tuple(tok.encode(get_parser("raw").parse([{"role": "user", "content": p}], add_generation_prompt=True)))
            for b in data[2:] for p in b["prompts"]}
    assert seen_second == want


def test_several_passes_per_batch_take_an_optimizer_step_each():
    log, s = [], _Scorer()
    _, cl = _cluster(2)
    learner = _learner(cl, s, log, algo={"num_iterations": 3})
    learner.train(_data(2))
    # per batch: one pass as the groups arrive (2 groups, one update each) + 2 further passes over both groups
    assert cl.global_steps == 2 and len(log) == 8
    assert cl.actor_trainer.train_steps == 2 * (2 + 2 * 2)


def test_running_ahead_generates_with_older_weights_and_stays_within_the_bound():
    log, s = [], _Scorer()
    _, cl = _cluster(3)
    learner = _learner(cl, s, log, off_policy_steps=1)
    versions = []
    inner = learner._process_group

    def spy(items, defer_logps=False):
        ex = inner(items, defer_logps)
        if ex is not None:
            versions.append((learner.policy_version, int(ex.policy_version)))
        return ex
    learner._process_group = spy
    learner.train(_data(3))
    assert cl.global_steps == 3 and learner.stale_dropped == 0
    assert all(0 <= now - gen <= 1 for now, gen in versions)


def test_groups_generated_too_long_ago_are_dropped():
    log, s = [], _Scorer()
    _, cl = _cluster(2)
    learner = _learner(cl, s, log)
    inner = learner._process_group

    def age(items, defer_logps=False):
        ex = inner(items, defer_logps)
        if ex is not None and learner.policy_version == 1:
            ex.policy_version = -1 if age.first else 0                           # unknown passes, an old version does not
            age.first = False
        return ex
    age.first = True
    learner._process_group = age
    learner.train(_data(2))
    assert learner.stale_dropped == 1 and cl.global_steps == 2


def test_group_without_signal_is_skipped_and_invalid_statuses_do_not_train():
    log = []
    flat = _Scorer(lambda ids, lens: [1.0] * len(lens))                           # equal rewards: zero advantages
    _, cl = _cluster(1)
    before = torch.cat([p.detach().reshape(-1).clone() for p in cl.train_actor.parameters()])
    _learner(cl, flat, log).train(_data(1))
    after = torch.cat([p.detach().reshape(-1) for p in cl.train_actor.parameters()])
    assert flat.calls == 2 and torch.allclose(before, after, atol=1e-7)           # zero advantages move nothing

    async def broken(**kw):
        raise RuntimeError("engine down")
    _, cl2 = _cluster(1)
    s = _Scorer()
    learner = AgenticGRPOLearner(cl2, [s], GRPOConfig(num_generations=2, beta=0.0), chat_parser=get_parser("raw"), model_client=broken)
    learner.train(_data(1))
    assert cl2.actor_trainer.train_steps == 0                                    # every episode failed: nothing to train on
    assert cl2.metrics_logger.get_metric("", "trajectory/valid_frac", "train") == 0.0


def test_eval_runs_on_its_cadence():
    log, s = [], _Scorer()
    _, cl = _cluster(2, eval_every=1)
    learner = _learner(cl, s, log)
    evals = []
    inner = learner.evaluate
    learner.evaluate = lambda ds: evals.append(cl.global_steps) or inner(ds)
    learner.train(_data(2), eval_ds=_data(1))
    assert evals == [1, 2]
    assert cl.metrics_logger.metric_exists("", "eval/rewards/mean", "eval")
    assert len(cl.metrics_logger.get_metric_history("", "eval/episodes", "eval")) == 2
