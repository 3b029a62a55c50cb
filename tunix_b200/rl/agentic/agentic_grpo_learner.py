"""Agentic GRPO learner (tunix/rl/agentic/agentic_grpo_learner.py:63-931): pads the multi-turn token / mask /
log-prob streams of a group, scores trajectories (environment reward + reward functions), computes
group-relative advantages and builds a `TrainExample` whose completion side is the whole conversation after
the first prompt, with environment tokens masked out of the loss."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ...common.datatypes import Mode
from .. import algo_core, common, function_registry
from ..algorithm_config import GRPOConfig
from .agentic_rl_learner import AgenticRLLearner
from .agents.agent_types import INVALID_TRAJECTORY_STATUSES


class AgenticGRPOLearner(AgenticRLLearner):
    def __init__(self, rl_cluster, reward_fns, algo_config: GRPOConfig, **kw):
        super().__init__(rl_cluster, reward_fns, algo_config, **kw)
        loss_fn = function_registry.get_policy_loss_fn(algo_config.policy_loss_fn)
        chunk = self.tcfg.compute_logps_chunk_size
        tr = rl_cluster.actor_trainer
        tr.with_loss_fn(lambda model, train_example: loss_fn(model, train_example, algo_config, self.pad_id, self.eos_id,
                                                             compute_logps_chunk_size=chunk), has_aux=True)
        tr.with_gen_model_input_fn(lambda ex: {"train_example": ex})
        tr.with_rl_metrics_to_log({k: np.mean for k in ("kl", "pg_clipfrac", "ppo_kl", "entropy")})
        self.advantage_fn = function_registry.get_advantage_estimator(algo_config.advantage_estimator)

    def _process_group(self, items: list, defer_logps: bool = False) -> Optional[common.TrainExample]:
        """`defer_logps`: leave the reference log-probs out; the caller computes them after packing."""
        cfg, dev = self.algo_config, self.device
        trajs = [it.traj for it in sorted(items, key=lambda x: x.episode_id)]
        valid = np.asarray([t["status"] not in INVALID_TRAJECTORY_STATUSES and t["conversation_masks"].sum() > 0
                            for t in trajs])
        rc = self.rl_cluster._rollout_config(Mode.TRAIN)
        P = max(max(len(t["prompt_tokens"]) for t in trajs), 1)
        C = max(max(len(t["conversation_tokens"]) for t in trajs), 1)
        G = len(trajs)
        pids = np.full((G, P), self.pad_id, np.int64)
        pmask = np.zeros((G, P), np.int32)
        cids = np.full((G, C), self.pad_id, np.int64)
        cmask = np.zeros((G, C), np.int32)
        old = np.zeros((G, C), np.float32)
        for i, t in enumerate(trajs):
            p, c = t["prompt_tokens"], t["conversation_tokens"]
            pids[i, P - len(p):], pmask[i, P - len(p):] = p, 1
            cids[i, :len(c)], cmask[i, :len(c)] = c, t["conversation_masks"]
            old[i, :len(c)] = t["old_logprobs"]
        env_r = np.asarray([t["trajectory_reward"] for t in trajs], np.float32)
        rewards = env_r
        if self.reward_manager is not None:
            tok = self.rl_cluster.tokenizer
            comps = [tok.decode([x for x in t["conversation_tokens"].tolist()]) for t in trajs]
            out = self.reward_manager([""] * G, comps, env_rewards=env_r, completion_ids=cids,
                                      completion_lengths=np.asarray([len(t["conversation_tokens"]) for t in trajs]))
            rewards = out["rewards"]
        adv = self.advantage_fn(rewards=rewards, num_generations=G, valid_mask=valid)
        cmask = cmask * valid[:, None].astype(np.int32)
        self.rl_cluster.buffer_metrics({
            "rewards/score/mean": (float(rewards.mean()), np.mean),
            "trajectory/valid_frac": (float(valid.mean()), np.mean),
            "trajectory/num_turns": (float(np.mean([t["num_turns"] for t in trajs])), np.mean),
            "completions/mean_length": (float(np.mean([len(t["conversation_tokens"]) for t in trajs])), np.mean)}, Mode.TRAIN)
        if cmask.sum() == 0:
            return None
        t_ = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
        # full token mask: environment tokens are real context (attended to) but carry no loss
        ex = common.TrainExample(prompt_ids=t_(pids), prompt_mask=t_(pmask), completion_ids=t_(cids),
                                 completion_mask=t_(cmask), advantages=t_(np.asarray(adv, np.float32)),
                                 old_per_token_logps=t_(old) if cfg.use_rollout_logps else None,
                                 policy_version=min((int(t["policy_version"]) for t in trajs if t.get("policy_version") is not None),
                                                    default=self.policy_version))
        if getattr(cfg, "beta", 0.0) != 0.0 and not defer_logps:
            ctx_mask = t_((cids != self.pad_id).astype(np.int32))
            ex.ref_per_token_logps = self.rl_cluster.get_ref_per_token_logps(
                ex.prompt_ids, ex.completion_ids, self.pad_id, self.eos_id, completion_mask=ctx_mask,
                temperature=cfg.temperature)
        ex.completion_attention_mask = t_((cids != self.pad_id).astype(np.int32))
        return ex
