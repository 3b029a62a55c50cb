"""RLCluster (alias RLEngine): owns the models of an RL job, their placement, the rollout engine, the
inference worker for frozen models and the trainers (tunix/rl/rl_cluster.py:102-1366).

One process per GPU. `ClusterConfig.role_to_mesh` maps each role to a mesh (a set of ranks); in the
colocated layout (all roles on all ranks, the default and the layout of the GRPO benchmark config) phases
alternate on the same GPUs: rollout -> reference / old log-probs -> actor update -> weight sync.

Weight sharing (:196-226): when the rollout model and the actor are the same object the sync is free; with
LoRA the reference policy is the actor with adapters disabled, so actor, reference and sampler share one
copy of the backbone. Otherwise `sync_weights` copies (LoRA-only when adapters exist) into the rollout
model; across ranks `rl/reshard.py` moves shards peer to peer.
"""
from __future__ import annotations

import contextlib
import gc
import itertools
import time
from typing import Any, Callable, Optional, Sequence

import numpy as np
import torch

from ..common.configs import ClusterConfig, RolloutConfig
from ..common.datatypes import Mode, Role
from ..lora import disable_adapters, is_lora_enabled, lora_state_dict
from ..sft import metrics_logger as ml
from . import common
from .inference.inference_worker import InferenceWorker
from .rollout.base_rollout import BaseRollout, RolloutOutput
from .rollout.vanilla_rollout import VanillaRollout
from .trainer import Trainer


class RLCluster:
    def __init__(self, *, actor, reference=None, critic=None, reward=None, rollout_model=None, tokenizer,
                 cluster_config: ClusterConfig, perf_tracer=None, metrics_logger: Optional[ml.MetricsLogger] = None):
        self.cluster_config = cluster_config
        self.tokenizer = tokenizer
        self.perf = perf_tracer
        tcfg = cluster_config.training_config
        self.train_actor = actor
        self.critic = critic
        self.reward = reward
        self._lora = is_lora_enabled(actor)
        # reference: explicit model, or the actor's frozen backbone when adapters are present
        self._ref_shares_backbone = reference is None and self._lora
        self.reference = reference
        self.rollout_actor = rollout_model if rollout_model is not None else actor
        self._rollout_shares_weights = self.rollout_actor is actor
        self.global_steps = 0
        self._buffered_metrics: dict = {}
        self._metrics_step = None
        self.metrics_logger = metrics_logger or ml.MetricsLogger(tcfg.metrics_logging_options)
        self._init_rollout()
        models = {}
        if self.reference is not None:
            models["reference"] = self.reference
        if critic is not None:
            models["critic"] = critic
        if reward is not None:
            models["reward"] = reward
        self.inference_worker = InferenceWorker(models)
        self._init_trainers()
        self._anchor = None   # pinned-host copy of the start-of-step policy (for off-policy old log-probs)

    # ----------------------------------------------------------------- setup
    def _rollout_config(self, mode=Mode.TRAIN) -> RolloutConfig:
        rc = self.cluster_config.rollout_config
        if isinstance(rc, dict):
            return rc.get(mode, rc.get(str(mode), next(iter(rc.values()))))
        return rc

    def _init_rollout(self) -> None:
        eng = self.cluster_config.rollout_engine
        rc = self._rollout_config()
        if isinstance(eng, BaseRollout):
            self.rollout = eng
        elif isinstance(eng, type) and issubclass(eng, BaseRollout):
            self.rollout = eng(model=self.rollout_actor, tokenizer=self.tokenizer, rollout_config=rc)
        elif eng in ("vanilla", "paged"):
            cache = max(rc.kv_cache_size, rc.max_prompt_length + rc.max_tokens_to_generate)
            self.rollout = VanillaRollout(self.rollout_actor, self.tokenizer, cache,
                                          engine="paged" if eng == "paged" else "dense")
        elif eng in ("vllm", "sglang_jax"):
            raise ValueError(f"rollout_engine={eng!r} belongs to the reference's TPU integrations; "
                             "use 'vanilla' or 'paged' (the in-framework engines)")
        else:
            raise ValueError(f"unknown rollout engine {eng!r}")

    def _init_trainers(self) -> None:
        import copy
        tcfg = self.cluster_config.training_config
        root = tcfg.checkpoint_root_directory

        def cfg_for(role: str):
            c = copy.copy(tcfg)
            if root:
                c.checkpoint_root_directory = f"{root}/{role}"
            c.metrics_prefix = role
            c.pbar_description = None
            return c

        self.actor_trainer = Trainer(self.train_actor, tcfg.actor_optimizer, cfg_for("actor"),
                                     metrics_logger=self.metrics_logger, perf_tracer=self.perf, role="actor")
        self.critic_trainer = None
        if self.critic is not None:
            opt = tcfg.critic_optimizer or copy.deepcopy(tcfg.actor_optimizer)
            self.critic_trainer = Trainer(self.critic, opt, cfg_for("critic"), metrics_logger=self.metrics_logger,
                                          perf_tracer=self.perf, role="critic")
        self.global_steps = self.actor_trainer.restored_global_step

    # -------------------------------------------------------------- generate
    def _span(self, name: str):
        return self.perf.span(name, device=True) if self.perf is not None else contextlib.nullcontext()

    def generate(self, prompts: Sequence[Any], mode=Mode.TRAIN, micro_batch_size: Optional[int] = None,
                 apply_chat_template: bool = False, prompt_token_ids: Optional[Sequence[Sequence[int]]] = None,
                 **kwargs) -> RolloutOutput:
        """Generate completions in micro-batches and merge them into one RolloutOutput."""
        rc = self._rollout_config(mode)
        if apply_chat_template and prompt_token_ids is None:
            prompts = [self.tokenizer.apply_chat_template([{"role": "user", "content": p}] if isinstance(p, str) else p,
                                                          add_generation_prompt=True, tokenize=False) for p in prompts]
        n = len(prompt_token_ids) if prompt_token_ids is not None else len(prompts)
        mb = micro_batch_size or n
        outs = []
        with self._span("rollout"):
            for s0 in range(0, n, mb):
                kw = dict(kwargs)
                if prompt_token_ids is not None:
                    kw["prompt_token_ids"] = prompt_token_ids[s0:s0 + mb]
                outs.append(self.rollout.generate(None if prompt_token_ids is not None else list(prompts[s0:s0 + mb]), rc, **kw))
        if len(outs) == 1:
            return outs[0]
        P = max(o.left_padded_prompt_tokens.shape[1] for o in outs)
        pad = self.rollout.pad_id()
        prm = np.concatenate([np.pad(o.left_padded_prompt_tokens, ((0, 0), (P - o.left_padded_prompt_tokens.shape[1], 0)),
                                     constant_values=pad) for o in outs])
        return RolloutOutput(
            text=list(itertools.chain.from_iterable(o.text for o in outs)), logits=None,
            tokens=list(itertools.chain.from_iterable(o.tokens for o in outs)), left_padded_prompt_tokens=prm,
            logprobs=(list(itertools.chain.from_iterable(o.logprobs for o in outs)) if outs[0].logprobs is not None else None),
            prompt_lengths=(np.concatenate([o.prompt_lengths for o in outs]) if outs[0].prompt_lengths is not None else None))

    # ---------------------------------------------------------------- logps
    def _mb_apply(self, fn: Callable, tensors: tuple, micro_batch_size: Optional[int]):
        n = tensors[0].shape[0]
        mb = micro_batch_size or n
        outs = [fn(*[t[s0:s0 + mb] if t is not None else None for t in tensors]) for s0 in range(0, n, mb)]
        return torch.cat(outs, 0)

    def get_ref_per_token_logps(self, prompt_tokens, completion_tokens, pad_id, eos_id, micro_batch_size=None,
                                completion_mask=None, **kw):
        chunk = self.cluster_config.training_config.compute_logps_chunk_size
        with self._span("refer_inference"):
            if self._ref_shares_backbone:
                def fn(p, c, m):
                    with disable_adapters(self.train_actor):
                        return common.compute_per_token_logps(self.train_actor, p, c, pad_id, eos_id, completion_mask=m,
                                                              stop_gradient=True, chunk_size=chunk, **kw)
            elif self.reference is not None:
                def fn(p, c, m):
                    return self.inference_worker.get_ref_per_token_logps(p, c, pad_id, eos_id, completion_mask=m,
                                                                         chunk_size=chunk, **kw)
            else:
                raise ValueError("no reference model: pass `reference=` or use a LoRA actor (shared backbone)")
            return self._mb_apply(fn, (prompt_tokens, completion_tokens, completion_mask), micro_batch_size)

    def get_old_per_token_logps(self, prompt_tokens, completion_tokens, micro_batch_size=None, completion_mask=None, **kw):
        """Log-probs under the rollout policy's weights (the sampler's model)."""
        with self._span("old_logps"):
            fn = lambda p, c, m: self.rollout.get_per_token_logps(p, c, m)  # noqa: E731
            return self._mb_apply(fn, (prompt_tokens, completion_tokens, completion_mask), micro_batch_size)

    def get_actor_per_token_logps(self, prompt_tokens, completion_tokens, pad_id, eos_id, micro_batch_size=None,
                                  completion_mask=None, **kw):
        chunk = self.cluster_config.training_config.compute_logps_chunk_size
        fn = lambda p, c, m: common.compute_per_token_logps(self.train_actor, p, c, pad_id, eos_id, completion_mask=m,  # noqa: E731
                                                            stop_gradient=True, chunk_size=chunk, **kw)
        return self._mb_apply(fn, (prompt_tokens, completion_tokens, completion_mask), micro_batch_size)

    def get_values(self, prompt_tokens, completion_tokens, pad_id, eos_id, micro_batch_size=None, completion_mask=None):
        fn = lambda p, c, m: self.inference_worker.get_values(p, c, pad_id, eos_id, m)  # noqa: E731
        return self._mb_apply(fn, (prompt_tokens, completion_tokens, completion_mask), micro_batch_size)

    def get_rewards(self, prompt_tokens, completion_tokens, pad_id, eos_id, micro_batch_size=None, completion_mask=None):
        fn = lambda p, c, m: self.inference_worker.get_rewards(p, c, pad_id, eos_id, m)  # noqa: E731
        return self._mb_apply(fn, (prompt_tokens, completion_tokens, completion_mask), micro_batch_size)

    # --------------------------------------------------------------- updates
    def update_actor(self, train_ds, eval_ds=None, skip_jit: bool = False) -> None:
        with self._span("actor_train"):
            # a checkpoint written during this update holds the weights of global step `global_steps` (0-based)
            self.actor_trainer.set_global_step(self.global_steps + 1)
            self.actor_trainer.train(train_ds, eval_ds, skip_jit)

    def update_critic(self, train_ds, eval_ds=None, skip_jit: bool = False) -> None:
        if self.critic_trainer is None:
            raise ValueError("no critic model")
        with self._span("critic_train"):
            self.critic_trainer.set_global_step(self.global_steps + 1)
            self.critic_trainer.train(train_ds, eval_ds, skip_jit)

    def sync_weights(self) -> None:
        """Push the actor's weights (LoRA-only when adapters exist) into the rollout engine; bump global step."""
        with self._span("weight_sync"):
            if not self._rollout_shares_weights:
                if self._lora:
                    self.rollout.update_params(lora_state_dict(self.train_actor))
                else:
                    self.rollout.update_params({n: p.detach() for n, p in self.train_actor.named_parameters()})
            if self.cluster_config.gc_collect_after_weight_sync:
                gc.collect()
        self.global_steps += 1

    def snapshot_anchor(self) -> None:
        """Pinned-host copy of the current policy (tunix/rl/rl_cluster.py:515-517,1297-1300)."""
        src = lora_state_dict(self.train_actor) if self._lora else dict(self.train_actor.named_parameters())
        self._anchor = {k: v.detach().to("cpu", copy=True).pin_memory() if torch.cuda.is_available()
                        else v.detach().clone() for k, v in src.items()}

    # --------------------------------------------------------------- offload
    def offload_to_host(self, role: str) -> None:
        """Move a model's weights to pinned host memory between phases (offload_to_cpu)."""
        m = {"actor": self.train_actor, "reference": self.reference, "critic": self.critic, "reward": self.reward}[role]
        if m is None:
            return
        for p in m.parameters():
            p.data = p.data.to("cpu").pin_memory() if torch.cuda.is_available() else p.data.cpu()

    def load_to_device(self, role: str, device) -> None:
        m = {"actor": self.train_actor, "reference": self.reference, "critic": self.critic, "reward": self.reward}[role]
        if m is None:
            return
        for p in m.parameters():
            p.data = p.data.to(device, non_blocking=True)

    # --------------------------------------------------------------- metrics
    def buffer_metrics(self, metrics: dict, mode=Mode.TRAIN, step: Optional[int] = None) -> None:
        """metrics: {name: (value(s), aggregation fn)}; flushed when the global step changes."""
        step = self.global_steps if step is None else step
        if self._metrics_step is not None and step != self._metrics_step:
            self.flush_metrics()
        self._metrics_step = step
        for k, (v, op) in metrics.items():
            slot = self._buffered_metrics.setdefault((k, str(mode)), ([], op))
            (slot[0].extend if isinstance(v, (list, tuple)) else slot[0].append)(v)

    def flush_metrics(self) -> None:
        for (k, mode), (vals, op) in self._buffered_metrics.items():
            vals = [v for v in vals if not isinstance(v, str)]
            if not vals:
                continue
            host = [float(v) if not isinstance(v, (list, np.ndarray)) else v for v in
                    [x.detach().float().cpu().numpy() if isinstance(x, torch.Tensor) else x for x in vals]]
            try:
                agg = op(host)
            except Exception:
                agg = float(np.mean(host))
            prefix, name = ("", k)
            self.metrics_logger.log(prefix, name, agg, mode, self._metrics_step)
        self._buffered_metrics = {}

    def close(self) -> None:
        self.flush_metrics()
        self.actor_trainer.close()
        if self.critic_trainer is not None:
            self.critic_trainer.close()


RLEngine = RLCluster
