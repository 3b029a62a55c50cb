"""GRPO learner (tunix/rl/grpo/grpo_learner.py:51-489) and its DAPO / Dr.GRPO variants
(tunix/rl/grpo/dapo_learner.py:28-161, drgrpo_learner.py:28-39).

Per prompt batch: rollout G completions per prompt -> right-pad completions -> reference log-probs (when
beta != 0) -> old-policy log-probs (the sampler's own log-probs, or a recompute under the rollout weights
when num_iterations > 1 or rollout log-probs are not trusted) -> rewards -> group-relative advantages ->
sampler/trainer agreement metrics -> TrainExample.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import numpy as np
import torch

from ...common.datatypes import Mode
from .. import algo_core, common, function_registry
from ..algorithm_config import GRPOConfig
from ..rl_cluster import RLCluster
from ..rl_learner import RLLearner

GrpoConfig = GRPOConfig


class GRPOLearner(RLLearner):
    def __init__(self, rl_cluster: RLCluster, reward_fns, algo_config: GRPOConfig, metric_fns=None,
                 data_shuffle_seed: Optional[int] = None):
        super().__init__(rl_cluster, algo_config, reward_fns, metric_fns, data_shuffle_seed)
        loss_fn = function_registry.get_policy_loss_fn(algo_config.policy_loss_fn)
        chunk = self.tcfg.compute_logps_chunk_size

        def loss(model, train_example):
            return loss_fn(model, train_example, algo_config, self.pad_id, self.eos_id, compute_logps_chunk_size=chunk,
                           loss_norm=self._loss_norm())

        tr = rl_cluster.actor_trainer
        tr.with_loss_fn(loss, has_aux=True)
        tr.with_gen_model_input_fn(lambda ex: {"train_example": ex})
        tr.with_rl_metrics_to_log({k: np.mean for k in ("kl", "kl_loss", "pg_clipfrac", "ppo_kl", "entropy",
                                                        "pg_clipfrac_lower", "is_ratio/mean", "is_ratio/max",
                                                        "advantage/abs_mean")})
        self.advantage_fn = function_registry.get_advantage_estimator(algo_config.advantage_estimator)

    def _loss_norm(self):
        if self.algo_config.loss_agg_mode == "sequence-mean-token-scale":
            return float(self.rl_cluster._rollout_config().max_tokens_to_generate)
        return None

    def _num_generations(self) -> int:
        return self.algo_config.num_generations

    def _num_iterations(self) -> int:
        return self.algo_config.num_iterations

    def _shape_rewards(self, rewards: np.ndarray, completions: list, lengths: np.ndarray) -> np.ndarray:
        return rewards

    def _generate_and_compute_advantage(self, training_input: dict, mode: Mode = Mode.TRAIN) -> common.TrainExample:
        cl, cfg = self.rl_cluster, self.algo_config
        dev = self.device
        prompts = training_input.get("prompts")
        ptoks = training_input.get("prompt_token_ids")
        rc = cl._rollout_config(mode)
        out = cl.generate(prompts, mode=mode, micro_batch_size=self.tcfg.rollout_micro_batch_size and
                          self.tcfg.rollout_micro_batch_size * cfg.num_generations, prompt_token_ids=ptoks)
        B = len(out.tokens)
        C = rc.max_tokens_to_generate
        comp = np.full((B, C), self.pad_id, np.int64)
        cmask = np.zeros((B, C), np.int32)
        lens = np.zeros(B, np.int64)
        for i, t in enumerate(out.tokens):
            n = min(len(t), C)
            comp[i, :n] = t[:n]
            cmask[i, :n] = 1
            lens[i] = n
        prompt_ids = torch.from_numpy(out.left_padded_prompt_tokens).to(dev)
        P = prompt_ids.shape[1]
        pl = out.prompt_lengths if out.prompt_lengths is not None else (out.left_padded_prompt_tokens != self.pad_id).sum(1)
        prompt_mask = (torch.arange(P, device=dev)[None] >= (P - torch.as_tensor(pl, device=dev))[:, None]).to(torch.int32)
        completion_ids = torch.from_numpy(comp).to(dev)
        completion_mask = torch.from_numpy(cmask).to(dev)
        mb = self.tcfg.compute_logps_micro_batch_size and self.tcfg.compute_logps_micro_batch_size * cfg.num_generations
        ref_logps = None
        if getattr(cfg, "beta", 0.0) != 0.0:
            ref_logps = cl.get_ref_per_token_logps(prompt_ids, completion_ids, self.pad_id, self.eos_id, mb,
                                                   completion_mask=completion_mask, temperature=cfg.temperature)
        old_logps = None
        if out.logprobs is not None and cfg.use_rollout_logps:
            ol = np.zeros((B, C), np.float32)
            for i, l in enumerate(out.logprobs):
                n = min(len(l), C)
                ol[i, :n] = np.asarray(l[:n], np.float32)
            old_logps = torch.from_numpy(ol).to(dev)
        elif cfg.num_iterations > 1 or not cfg.use_rollout_logps:
            old_logps = cl.get_old_per_token_logps(prompt_ids, completion_ids, mb, completion_mask=completion_mask)
        extra = {k: v for k, v in training_input.items() if k not in ("prompts", "prompt_token_ids")}
        prompt_texts = prompts if prompts is not None else [""] * B
        rewards = self._compute_rewards(list(prompt_texts), list(out.text), mode, completion_ids=comp,
                                        completion_lengths=lens, **extra)
        rewards = self._shape_rewards(np.asarray(rewards, np.float32), out.text, lens)
        adv = self.advantage_fn(rewards=rewards, num_generations=cfg.num_generations)
        cl.buffer_metrics({"completions/mean_length": (float(lens.mean()), np.mean),
                           "completions/max_length": (float(lens.max()), np.max),
                           "completions/min_length": (float(lens.min()), np.min)}, mode)
        for fn in self.metric_fns:
            cl.buffer_metrics(fn(prompts=prompt_texts, completions=out.text, rewards=rewards, advantages=adv), mode)
        # router replay: the experts the sampler chose, laid out over the padded [prompt | completion] stream
        routed = common.align_routed_experts(out.routed_experts, lens, P, C) if getattr(out, "routed_experts", None) else None
        return common.TrainExample(prompt_ids=prompt_ids, prompt_mask=prompt_mask, completion_ids=completion_ids,
                                   completion_mask=completion_mask,
                                   advantages=torch.from_numpy(np.asarray(adv, np.float32)).to(dev),
                                   ref_per_token_logps=ref_logps, old_per_token_logps=old_logps,
                                   routed_experts=None if routed is None else torch.from_numpy(routed).to(dev))


GrpoLearner = GRPOLearner


def __getattr__(name):
    """The DAPO and Dr. GRPO learners have modules of their own; they stay importable from here."""
    if name == "DAPOLearner":
        from .dapo_learner import DAPOLearner
        return DAPOLearner
    if name == "DrGRPOLearner":
        from .drgrpo_learner import DrGRPOLearner
        return DrGRPOLearner
    raise AttributeError(name)
