"""PPO learner (tunix/rl/ppo/ppo_learner.py:49-547): critic + optional reward model, token-level rewards
(sequence score at the last token minus beta * KL to the reference), GAE, actor and critic updates."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ...common.datatypes import Mode
from .. import algo_core, common, function_registry
from ..algorithm_config import PPOConfig
from ..rl_cluster import RLCluster
from ..rl_learner import RLLearner

PpoConfig = PPOConfig


class PPOLearner(RLLearner):
    def __init__(self, rl_cluster: RLCluster, ppo_config: PPOConfig, reward_fns=None, metric_fns=None,
                 data_shuffle_seed: Optional[int] = None):
        if rl_cluster.critic is None:
            raise ValueError("PPO needs a critic model")
        if reward_fns is None and rl_cluster.reward is None:
            raise ValueError("PPO needs reward functions or a reward model")
        super().__init__(rl_cluster, ppo_config, reward_fns, metric_fns, data_shuffle_seed)
        pol = function_registry.get_policy_loss_fn(ppo_config.policy_loss_fn)
        val = function_registry.get_value_loss_fn(ppo_config.value_loss_fn)
        rl_cluster.actor_trainer.with_loss_fn(
            lambda model, train_example: pol(model, train_example, ppo_config, self.pad_id, self.eos_id), has_aux=True)
        rl_cluster.actor_trainer.with_gen_model_input_fn(lambda ex: {"train_example": ex})
        rl_cluster.critic_trainer.with_loss_fn(
            lambda model, train_example: val(model, train_example, ppo_config, self.pad_id, self.eos_id), has_aux=True)
        rl_cluster.critic_trainer.with_gen_model_input_fn(lambda ex: {"train_example": ex})
        rl_cluster.actor_trainer.with_rl_metrics_to_log({k: np.mean for k in ("pg_clipfrac", "ppo_kl", "loss/entropy")})
        rl_cluster.critic_trainer.with_rl_metrics_to_log({k: np.mean for k in ("vf_clipfrac", "values/mean")})

    def _num_generations(self) -> int:
        return 1

    def _num_iterations(self) -> int:
        return self.algo_config.num_iterations

    def _train_on(self, examples) -> None:
        exs = list(examples)
        if not exs:
            return
        self.rl_cluster.update_actor(iter(exs), None)
        self.rl_cluster.update_critic(iter(exs), None)

    def _generate_and_compute_advantage(self, training_input: dict, mode: Mode = Mode.TRAIN) -> common.TrainExample:
        cl, cfg, dev = self.rl_cluster, self.algo_config, self.device
        prompts, ptoks = training_input.get("prompts"), training_input.get("prompt_token_ids")
        rc = cl._rollout_config(mode)
        out = cl.generate(prompts, mode=mode, micro_batch_size=self.tcfg.rollout_micro_batch_size, prompt_token_ids=ptoks)
        B, C = len(out.tokens), rc.max_tokens_to_generate
        comp = np.full((B, C), self.pad_id, np.int64)
        cmask = np.zeros((B, C), np.int32)
        lens = np.zeros(B, np.int64)
        for i, t in enumerate(out.tokens):
            n = min(len(t), C)
            comp[i, :n], cmask[i, :n], lens[i] = t[:n], 1, n
        prompt_ids = torch.from_numpy(out.left_padded_prompt_tokens).to(dev)
        P = prompt_ids.shape[1]
        pl = out.prompt_lengths if out.prompt_lengths is not None else (out.left_padded_prompt_tokens != self.pad_id).sum(1)
        prompt_mask = (torch.arange(P, device=dev)[None] >= (P - torch.as_tensor(pl, device=dev))[:, None]).to(torch.int32)
        completion_ids, completion_mask = torch.from_numpy(comp).to(dev), torch.from_numpy(cmask).to(dev)
        mb = self.tcfg.compute_logps_micro_batch_size
        old_logps = cl.get_old_per_token_logps(prompt_ids, completion_ids, mb, completion_mask=completion_mask)
        values = cl.get_values(prompt_ids, completion_ids, self.pad_id, self.eos_id, mb, completion_mask=completion_mask)
        values = values * completion_mask
        if cl.reward is not None:
            score = cl.get_rewards(prompt_ids, completion_ids, self.pad_id, self.eos_id, mb, completion_mask=completion_mask)
            score = score.float()
        else:
            extra = {k: v for k, v in training_input.items() if k not in ("prompts", "prompt_token_ids")}
            score = torch.from_numpy(self._compute_rewards(list(prompts or [""] * B), list(out.text), mode, completion_ids=comp,
                                                            completion_lengths=lens, **extra)).to(dev)
        rewards = torch.zeros(B, C, device=dev)
        last = torch.as_tensor(np.maximum(lens - 1, 0), device=dev)
        rewards[torch.arange(B, device=dev), last] = score
        if cfg.beta != 0.0 and (cl.reference is not None or cl._ref_shares_backbone):
            ref = cl.get_ref_per_token_logps(prompt_ids, completion_ids, self.pad_id, self.eos_id, mb,
                                             completion_mask=completion_mask)
            kl = common.compute_kl_divergence(old_logps, ref, cfg.kl_method, cfg.kl_clamp_value)
            rewards = rewards - cfg.beta * kl * completion_mask
            cl.buffer_metrics({"reward_kl_penalty": (float((kl * completion_mask).sum() / completion_mask.sum().clamp(min=1)), np.mean)}, mode)
        adv, returns = algo_core.compute_gae_advantages(rewards, values, completion_mask, cfg.gamma, cfg.gae_lambda)
        m = completion_mask.float()
        cl.buffer_metrics({"score/mean": (float(score.mean()), np.mean),
                           "advantages/mean": (float(algo_core.masked_mean(adv, m)), np.mean),
                           "returns/mean": (float(algo_core.masked_mean(returns, m)), np.mean),
                           "values/mean": (float(algo_core.masked_mean(values, m)), np.mean),
                           "completions/mean_length": (float(lens.mean()), np.mean)}, mode)
        return common.TrainExample(prompt_ids=prompt_ids, prompt_mask=prompt_mask, completion_ids=completion_ids,
                                   completion_mask=completion_mask, advantages=adv, old_per_token_logps=old_logps,
                                   returns=returns, old_values=values)


PpoLearner = PPOLearner
