"""End-to-end learner runs on tiny models (CPU): GRPO with the real sampler, PPO with a critic."""
import numpy as np
import torch

from tunix_b200 import optim
from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
from tunix_b200.lora import LoraProvider, apply_lora_to_model
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model
from tunix_b200.rl import utils as rl_utils
from tunix_b200.rl.algorithm_config import GRPOConfig, PPOConfig
from tunix_b200.rl.grpo.grpo_learner import GRPOLearner
from tunix_b200.rl.ppo.ppo_learner import PPOLearner
from tunix_b200.rl.rl_cluster import RLCluster
from tests.test_sampler_cpu import CharTok


def _cfg():
    return ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2,
                                            head_dim=16, num_kv_heads=1)


def reward_mod7(prompts, completions, completion_ids=None, completion_lengths=None, **kw):
    out = []
    for ids, n in zip(completion_ids, completion_lengths):
        ids = ids[:n]
        out.append(float((ids % 7 == 0).mean()) - 0.001 * n if n else 0.0)
    return out


def _cluster(actor, critic=None, reference=None, steps=2, tmp=None, mini=4, micro=2):
    tc = RLTrainingConfig(eval_every_n_steps=1000, max_steps=steps, actor_optimizer=optim.AdamW(1e-3),
                          critic_optimizer=optim.AdamW(1e-3), mini_batch_size=mini, train_micro_batch_size=micro,
                          checkpoint_root_directory=tmp)
    rc = RolloutConfig(max_tokens_to_generate=6, max_prompt_length=8, temperature=1.0, top_p=1.0, seed=3,
                       kv_cache_size=32, eos_tokens=[63])
    cc = ClusterConfig(role_to_mesh={}, training_config=tc, rollout_config=rc)
    return RLCluster(actor=actor, reference=reference, critic=critic, tokenizer=CharTok(), cluster_config=cc)


def test_grpo_learner_runs_and_updates_lora_only(tmp_path):
    actor = create_model(_cfg(), seed=0)
    apply_lora_to_model(actor, LoraProvider(module_path=r".*(q_proj|v_proj)", rank=4, alpha=8.0))
    before = {n: p.detach().clone() for n, p in actor.named_parameters()}
    cl = _cluster(actor, tmp=str(tmp_path))
    learner = GRPOLearner(cl, [reward_mod7], GRPOConfig(num_generations=2, beta=0.04))
    data = [{"prompts": ["ab", "cd", "ef", "gh"]} for _ in range(2)]
    learner.train(data)
    assert cl.global_steps == 2
    changed = [n for n, p in actor.named_parameters() if not torch.equal(p, before[n])]
    assert changed and all("lora" in n for n in changed)
    hist = cl.metrics_logger.get_metric_history("", "rewards/score/mean", "train")
    assert len(hist) == 2
    assert cl.metrics_logger.metric_exists("actor", "kl", "train")
    # resume: the actor checkpoint carries the global step
    actor2 = create_model(_cfg(), seed=0)
    apply_lora_to_model(actor2, LoraProvider(module_path=r".*(q_proj|v_proj)", rank=4, alpha=8.0))
    cl2 = _cluster(actor2, tmp=str(tmp_path))
    assert cl2.global_steps == 2
    cl2.close()


def test_learner_reports_the_layouts_perf_metrics_every_step():
    from tunix_b200.perf.trace import PerfTracer
    actor = create_model(_cfg(), seed=0)
    ref = create_model(_cfg(), seed=0)
    tc = RLTrainingConfig(eval_every_n_steps=1000, max_steps=2, actor_optimizer=optim.AdamW(1e-3), mini_batch_size=4,
                          train_micro_batch_size=2)
    rc = RolloutConfig(max_tokens_to_generate=6, max_prompt_length=8, temperature=1.0, top_p=1.0, seed=3,
                       kv_cache_size=32, eos_tokens=[63])
    tracer = PerfTracer()
    cl = RLCluster(actor=actor, reference=ref, tokenizer=CharTok(), perf_tracer=tracer, separate_rollout_copy=True,
                   cluster_config=ClusterConfig(role_to_mesh={}, training_config=tc, rollout_config=rc))
    GRPOLearner(cl, [reward_mod7], GRPOConfig(num_generations=2, beta=0.04)).train(
        [{"prompts": ["ab", "cd", "ef", "gh"]} for _ in range(2)])
    lg = cl.metrics_logger
    steps = lg.get_metric_history("", "perf/global_step_time", "train")
    assert len(steps) == 2 and all(t > 0 for t in steps)
    for name in ("perf/sum/rollout_time", "perf/sum/refer_inference_time", "perf/sum/actor_train_time", "perf/weight_sync_time"):
        assert lg.get_metric_history("", name, "train")[-1] > 0, name
    assert lg.get_metric_history("", "perf/global_step_time", "train")[-1] >= \
        lg.get_metric_history("", "perf/sum/actor_train_time", "train")[-1]
    # the sampler's own copy follows the actor
    a = torch.cat([p.detach().reshape(-1) for p in actor.parameters()])
    r = torch.cat([p.detach().reshape(-1) for p in cl.rollout_actor.parameters()])
    assert cl.rollout_actor is not actor and torch.equal(a, r)


def test_grpo_full_weight_with_reference_and_gspo():
    actor = create_model(_cfg(), seed=0)
    ref = create_model(_cfg(), seed=0)
    cl = _cluster(actor, reference=ref, steps=1)
    learner = GRPOLearner(cl, [reward_mod7], GRPOConfig(num_generations=2, beta=0.04, loss_algo="gspo-token",
                                                        num_iterations=2))
    learner.train([{"prompts": ["ab", "cd", "ef", "gh"]}])
    assert cl.global_steps == 1
    assert cl.actor_trainer.train_steps == 2          # mu = 2 iterations over the same rollouts


def test_ppo_learner_runs():
    actor = create_model(_cfg(), seed=0)
    critic = rl_utils.create_critic_model(actor)
    ref = create_model(_cfg(), seed=0)
    cl = _cluster(actor, critic=critic, reference=ref, steps=1)
    learner = PPOLearner(cl, PPOConfig(), reward_fns=[reward_mod7])
    learner.train([{"prompts": ["ab", "cd", "ef", "gh"]}])
    assert cl.global_steps == 1
    assert cl.critic_trainer.train_steps == 1


def test_micro_batch_items_are_merged_to_the_service_target_and_every_pass_ends_with_an_update():
    """A dataset that yields micro-batches of 2 prompts, mini-batch 4, rollout micro-batch 4: two items are merged into
    one generate-and-score pass; the step's micro-batches carry explicit update flags (last one always updates)."""
    actor = create_model(_cfg(), seed=0)
    ref = create_model(_cfg(), seed=0)
    tc = RLTrainingConfig(eval_every_n_steps=1000, max_steps=2, actor_optimizer=optim.AdamW(1e-3), mini_batch_size=4,
                          train_micro_batch_size=1, rollout_micro_batch_size=4, compute_logps_micro_batch_size=2)
    rc = RolloutConfig(max_tokens_to_generate=6, max_prompt_length=8, temperature=1.0, top_p=1.0, seed=3, kv_cache_size=32,
                       eos_tokens=[63])
    cl = RLCluster(actor=actor, reference=ref, tokenizer=CharTok(),
                   cluster_config=ClusterConfig(role_to_mesh={}, training_config=tc, rollout_config=rc))
    learner = GRPOLearner(cl, [reward_mod7], GRPOConfig(num_generations=2, beta=0.04))
    calls = []
    orig = learner._generate_and_compute_advantage

    def spy(batch, mode=None):
        calls.append(len(batch["prompts"]))
        return orig(batch, mode)
    learner._generate_and_compute_advantage = spy
    flags = []
    orig_train = cl.actor_trainer._train_step

    def spy_step(batch, is_update):
        flags.append(bool(is_update))
        return orig_train(batch, is_update)
    cl.actor_trainer._train_step = spy_step
    assert learner._service_target() == 4
    learner.train([{"prompts": [f"{chr(97 + i)}b", f"{chr(98 + i)}c"]} for i in range(4)])      # 4 items of 2 prompts
    assert cl.global_steps == 2 and calls == [8, 8]             # 2 items x 2 prompts x G per pass
    assert flags == [False, False, False, True] * 2             # 4 micro-batches of 1 prompt x G, accumulation 4
    assert cl.actor_trainer.train_steps == 2


def test_grpo_on_a_moe_actor_replays_the_samplers_routing():
    """`return_routed_experts` on the rollout config: the dense sampler records every token's experts, the learner lays
    them out over the padded stream and the update's forward pass is routed exactly as the sampler was."""
    cfg = _cfg().replace(num_experts=4, num_experts_per_tok=2, moe_hidden_dim=32)
    actor = create_model(cfg, seed=0)
    ref = create_model(cfg, seed=0)
    tc = RLTrainingConfig(eval_every_n_steps=1000, max_steps=1, actor_optimizer=optim.AdamW(1e-3), mini_batch_size=2,
                          train_micro_batch_size=2)
    rc = RolloutConfig(max_tokens_to_generate=5, max_prompt_length=8, temperature=1.0, top_p=1.0, seed=3, kv_cache_size=32,
                       eos_tokens=[63], return_routed_experts=True)
    cl = RLCluster(actor=actor, reference=ref, tokenizer=CharTok(),
                   cluster_config=ClusterConfig(role_to_mesh={}, training_config=tc, rollout_config=rc))
    out = cl.generate(["abc", "de"])
    assert out.routed_experts is not None and len(out.routed_experts) == 2
    for r_, t_, pl in zip(out.routed_experts, out.tokens, out.prompt_lengths):
        assert r_.shape == (int(pl) + len(t_) - 1, 1, 2) and r_.min() >= 0 and r_.max() < 4
    learner = GRPOLearner(cl, [reward_mod7], GRPOConfig(num_generations=2, beta=0.04))
    seen = []
    orig = actor.forward

    def spy(*a, **kw):
        if kw.get("routed_experts") is not None and torch.is_grad_enabled():
            seen.append(kw["routed_experts"].clone())
        return orig(*a, **kw)
    actor.forward = spy
    learner.train([{"prompts": ["ab", "cd"]}])
    assert cl.global_steps == 1 and seen and seen[0].dim() == 4 and int(seen[0].max()) < 4
    assert (seen[0] == -1).any()                  # padding slots are left to the model's own router


def test_step_timelines_are_written_as_a_trace_per_step(tmp_path):
    import json
    from tunix_b200.common.configs import PerfMetricsOptions
    from tunix_b200.perf.trace import PerfTracer
    actor = create_model(_cfg(), seed=0)
    tc = RLTrainingConfig(eval_every_n_steps=1000, max_steps=2, actor_optimizer=optim.AdamW(1e-3), mini_batch_size=4, train_micro_batch_size=2,
                          perf_metrics_options=PerfMetricsOptions(enable_perf_v2=True, enable_trace_writer=True, log_dir=str(tmp_path)))
    rc = RolloutConfig(max_tokens_to_generate=6, max_prompt_length=8, temperature=1.0, top_p=1.0, seed=3, kv_cache_size=32, eos_tokens=[63])
    cl = RLCluster(actor=actor, tokenizer=CharTok(), perf_tracer=PerfTracer(),
                   cluster_config=ClusterConfig(role_to_mesh={}, training_config=tc, rollout_config=rc))
    learner = GRPOLearner(cl, [reward_mod7], GRPOConfig(num_generations=2, beta=0.0))
    learner.train([{"prompts": ["ab", "cd", "ef", "gh"]} for _ in range(2)])
    learner._trace_exporter.close()
    assert len(learner._trace_exporter.timelines) >= 1
    hosts = [tl for tid, tl in learner._trace_exporter.timelines.items() if tid.startswith("host-")]
    assert len(hosts) == 2 and all(len(tl.committed_steps) == 2 for tl in hosts)   # trainer thread and rollout producer; a step each per global step
    names = {s.name for tl in hosts for step in tl.committed_steps for s in step.values()}
    assert {"global_step", "rollout", "actor_train"} <= names
    ev = json.load(open(learner._trace_exporter.trace_file_path))["traceEvents"]
    slices = [e for e in ev if e["ph"] == "X"]
    assert any(e["name"].startswith("rollout") for e in slices) and any("step=1" in e["name"] for e in slices)
