"""RLCluster (alias RLEngine): owns the models of an RL job, their placement, the rollout engine, the
inference worker for frozen models and the trainers (tunix/rl/rl_cluster.py:102-1366).

One process per GPU. `ClusterConfig.role_to_mesh` maps each role to a mesh (a set of ranks,
`rl/placement.py`). Every rank of the job constructs an `RLCluster` with the models of the roles it hosts:

* colocated (all roles on the actor's ranks, the default and the layout of the GRPO benchmark config): phases
  alternate on the same GPUs: rollout -> reference / old log-probs -> actor update -> weight sync. Every rank is
  a data-parallel replica of the loop over its own prompts.
* disaggregated (rollout, and possibly the reference, on other ranks than the actor): the actor's ranks run the
  loop; the other ranks call `serve()` and answer rounds of work (`generate`, `ref_logps`), see
  `placement.RoleExchange`. `generate_begin` opens a round early so that generation of the next batch runs while
  the actor trains on the current one.

What the mesh of a role asks for is applied here (the reference's `_load_model` reshards every model onto its
mesh, :228-287): an `fsdp` axis turns the actor's AdamW into the sharded optimizer over that group and stores a
frozen reference / critic / reward model as row blocks whose GEMMs gather them on use (`parallel/fsdp3.py`,
forward only); a `tp` axis slices the actor with `parallel/tp.py`.

Weight sharing (:196-226): when the rollout model and the actor are the same object the sync is free; with
LoRA the reference policy is the actor with adapters disabled, so actor, reference and sampler share one
copy of the backbone. Otherwise `sync_weights` moves the actor's weights into the sampler's own copy with
`rl/reshard.py`: the source ranks stage, the rollout ranks pull their rectangles peer to peer, whatever the two
layouts are (the same call serves the colocated separate-copy case, where every pull is local).
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
from .placement import RoleExchange, RolePlacement
from .inference.inference_worker import InferenceWorker
from .rollout.base_rollout import BaseRollout, RolloutOutput
from .rollout.vanilla_rollout import VanillaRollout
from .trainer import Trainer


class RLCluster:
    def __init__(self, *, actor=None, reference=None, critic=None, reward=None, rollout_model=None, tokenizer,
                 cluster_config: ClusterConfig, perf_tracer=None, metrics_logger: Optional[ml.MetricsLogger] = None,
                 placement: Optional[RolePlacement] = None, separate_rollout_copy: bool = False):
        """`actor` ... `rollout_model`: the models of the roles THIS rank hosts (None for the others; a rollout
        rank of a disaggregated job passes `rollout_model` only). `separate_rollout_copy`: in the colocated layout
        give the sampler its own copy of the weights, refreshed by `sync_weights`, instead of sharing the actor's."""
        self.cluster_config = cluster_config
        self.tokenizer = tokenizer
        self.perf = perf_tracer
        tcfg = cluster_config.training_config
        self.placement = placement or RolePlacement(cluster_config.role_to_mesh)
        pl = self.placement
        self.exchange = RoleExchange(pl, on_sync=self._transfer_weights)
        self.is_controller = pl.is_controller
        if pl.has(Role.ACTOR) and actor is None:
            raise ValueError(f"rank {pl.rank} hosts the actor (ranks {pl.ranks(Role.ACTOR)}) but got no actor model")
        if not pl.has(Role.ACTOR):
            actor = None
        self.train_actor = actor
        self.critic = critic if pl.has(Role.CRITIC) else None
        self.reward = reward if pl.has(Role.REWARD) else None
        self._lora = actor is not None and is_lora_enabled(actor)
        # reference: explicit model, or the actor's frozen backbone when adapters are present
        self._ref_shares_backbone = reference is None and self._lora and pl.same(Role.REFERENCE, Role.ACTOR)
        self.reference = reference if pl.has(Role.REFERENCE) else None
        if pl.has(Role.ROLLOUT):
            if rollout_model is None and actor is not None and separate_rollout_copy:
                import copy
                rollout_model = copy.deepcopy(actor)
                for p in rollout_model.parameters():
                    p.requires_grad_(False)
            if rollout_model is None and actor is None:
                raise ValueError(f"rank {pl.rank} hosts the rollout role but got neither a rollout model nor an actor")
            self.rollout_actor = rollout_model if rollout_model is not None else actor
        else:
            self.rollout_actor = None
        self._rollout_shares_weights = self.rollout_actor is not None and self.rollout_actor is actor and \
            pl.same(Role.ROLLOUT, Role.ACTOR)
        self.global_steps = 0
        self.last_weight_sync_seconds: Optional[float] = None
        self.last_weight_sync_bytes = 0
        self._resharder = None
        self._resharder_key = None
        self._prefetch = None
        self.actor_trainer = self.critic_trainer = None
        if pl.world > 1 and not pl.same(Role.ROLLOUT, Role.ACTOR) and torch.cuda.is_available() and \
                all(pl.axis_size(r, "tp") <= 1 for r in (Role.ACTOR, Role.ROLLOUT)):
            # The cross-rank weight transfer allocates symmetric memory over ALL ranks. It is set up (and run once)
            # here, before the trainer ranks allocate symmetric memory among themselves (sharded optimizer, sharded
            # reference): on 4 GPUs (2 trainers + 2 samplers) every rank was found waiting in the symmetric-memory
            # rendezvous of the transfer's staging buffer when that rendezvous came after the trainers' own ones,
            # i.e. after the ranks had taken part in different numbers of rendezvous.
            self._transfer_weights()
        self._apply_mesh_strategies()
        self._buffered_metrics: dict = {}
        self._metrics_step = None
        self.metrics_logger = metrics_logger or ml.MetricsLogger(tcfg.metrics_logging_options)
        self.rollout = None
        if self.rollout_actor is not None:
            self._init_rollout()
        models = {}
        if self.reference is not None:
            models["reference"] = self.reference
        if self.critic is not None:
            models["critic"] = self.critic
        if self.reward is not None:
            models["reward"] = self.reward
        self.inference_worker = InferenceWorker(models)
        if self.train_actor is not None:
            self._init_trainers()
        self._anchor = None   # pinned-host copy of the start-of-step policy (for off-policy old log-probs)
        self.exchange.register(Role.ROLLOUT, "generate", self._serve_generate)
        self.exchange.register(Role.REFERENCE, "ref_logps", self._serve_ref_logps)

    def _apply_mesh_strategies(self) -> None:
        """Turn the axes of each role's mesh into the parallel form of the model this rank holds."""
        pl, tcfg = self.placement, self.cluster_config.training_config
        if self.train_actor is not None:
            tp = pl.axis_size(Role.ACTOR, "tp")
            if tp > 1 and getattr(self.train_actor, "tp", None) is None:
                from ..parallel import tp as tp_lib
                dev = next(self.train_actor.parameters()).device
                tp_lib.apply_tensor_parallel(self.train_actor, tp_lib.TPContext(group=pl.axis_group(Role.ACTOR, "tp"),
                                                                                device=dev))
            if pl.axis_size(Role.ACTOR, "fsdp") > 1 and tcfg.actor_optimizer is not None:
                from ..parallel import fsdp
                tcfg.actor_optimizer = fsdp.shard_optimizer(tcfg.actor_optimizer, pl.axis_group(Role.ACTOR, "fsdp"))
        if self.rollout_actor is not None and self.rollout_actor is not self.train_actor:
            # a rollout mesh with a `tp` axis: the sampler's copy is sliced over it and decodes tensor-parallel; the
            # ranks of one tp group receive the same requests from the exchange
            tp = pl.axis_size(Role.ROLLOUT, "tp")
            if tp > 1 and getattr(self.rollout_actor, "tp", None) is None:
                from ..parallel import tp as tp_lib
                dev = next(self.rollout_actor.parameters()).device
                tp_lib.apply_tensor_parallel(self.rollout_actor, tp_lib.TPContext(group=pl.axis_group(Role.ROLLOUT, "tp"),
                                                                                  device=dev))
        if getattr(self.cluster_config, "shard_frozen_models", True):
            for role, model in ((Role.REFERENCE, self.reference), (Role.CRITIC, None), (Role.REWARD, self.reward)):
                if model is None or pl.axis_size(role, "fsdp") <= 1 or getattr(model, "dp_shard", None) is not None:
                    continue
                if any(p.requires_grad for p in model.parameters()) or not hasattr(model, "layers"):
                    continue
                from ..parallel import fsdp3
                dev = next(model.parameters()).device
                fsdp3.apply_weight_sharding(model, fsdp3.CommContext(group=pl.axis_group(role, "fsdp"), device=dev))

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
                                          engine="paged" if eng == "paged" else "dense", rollout_config=rc)
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
        """Generate completions in micro-batches and merge them into one RolloutOutput. When the rollout role sits
        on other ranks the prompts travel there in a round (or the round opened by `generate_begin` is closed)."""
        if not self.exchange.is_local(Role.ROLLOUT):
            return self._generate_remote(prompts, mode, micro_batch_size, apply_chat_template, prompt_token_ids, kwargs)
        return self._generate_local(prompts, mode, micro_batch_size, apply_chat_template, prompt_token_ids, **kwargs)

    def _generate_local(self, prompts, mode=Mode.TRAIN, micro_batch_size=None, apply_chat_template=False,
                        prompt_token_ids=None, **kwargs) -> RolloutOutput:
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

    # -------------------------------------------------- generation on other ranks
    @staticmethod
    def _split_output(out: RolloutOutput) -> list:
        n = len(out.tokens)
        return [{"text": out.text[i], "tokens": np.asarray(out.tokens[i]),
                 "prompt": np.asarray(out.left_padded_prompt_tokens[i]),
                 "logprobs": None if out.logprobs is None else np.asarray(out.logprobs[i]),
                 "plen": None if out.prompt_lengths is None else int(out.prompt_lengths[i])} for i in range(n)]

    def _merge_output(self, rows: list) -> RolloutOutput:
        P = max(len(r["prompt"]) for r in rows)
        pad = self.tokenizer.pad_id()
        prm = np.stack([np.pad(r["prompt"], (P - len(r["prompt"]), 0), constant_values=pad) for r in rows])
        return RolloutOutput(text=[r["text"] for r in rows], logits=None, tokens=[r["tokens"] for r in rows],
                             left_padded_prompt_tokens=prm,
                             logprobs=None if rows[0]["logprobs"] is None else [r["logprobs"] for r in rows],
                             prompt_lengths=None if rows[0]["plen"] is None else np.asarray([r["plen"] for r in rows]))

    def _serve_generate(self, items: list) -> list:
        """Rollout ranks: one engine call per group of items that share their settings."""
        out: list = [None] * len(items)
        groups: dict = {}
        for i, it in enumerate(items):
            groups.setdefault((it["mode"], it["mb"], it["ids"] is not None), []).append(i)
        for (mode, mb, by_ids), idx in groups.items():
            prompts = None if by_ids else [items[i]["prompt"] for i in idx]
            ids = [items[i]["ids"] for i in idx] if by_ids else None
            res = self._generate_local(prompts, Mode(mode), mb, False, ids)     # records its own "rollout" span
            for i, row in zip(idx, self._split_output(res)):
                out[i] = row
        return out

    def _generate_items(self, prompts, mode, micro_batch_size, apply_chat_template, prompt_token_ids) -> list:
        if apply_chat_template and prompt_token_ids is None:
            prompts = [self.tokenizer.apply_chat_template([{"role": "user", "content": p}] if isinstance(p, str) else p,
                                                          add_generation_prompt=True, tokenize=False) for p in prompts]
        n = len(prompt_token_ids) if prompt_token_ids is not None else len(prompts)
        return [{"mode": str(mode), "mb": micro_batch_size, "prompt": None if prompt_token_ids is not None else prompts[i],
                 "ids": None if prompt_token_ids is None else [int(t) for t in prompt_token_ids[i]]} for i in range(n)]

    def generate_begin(self, prompts, mode=Mode.TRAIN, micro_batch_size=None, apply_chat_template: bool = False,
                       prompt_token_ids=None) -> bool:
        """Open the generation round for these prompts now and return; the matching `generate(...)` call (same
        prompts) collects the result. Between the two this rank is free to train while the rollout ranks work.
        No-op (False) when the rollout role is local."""
        if self.exchange.is_local(Role.ROLLOUT):
            return False
        self.generate_finish()
        items = self._generate_items(prompts, mode, micro_batch_size, apply_chat_template, prompt_token_ids)
        self._prefetch = {"items": items, "round": self.exchange.begin(Role.ROLLOUT, "generate", items), "rows": None}
        return True

    def generate_finish(self) -> None:
        """Close an open generation round (its results are kept for the `generate` call that asks for them)."""
        pf = self._prefetch
        if pf is not None and pf["round"] is not None:
            pf["rows"] = self.exchange.end(pf["round"])
            pf["round"] = None

    def _generate_remote(self, prompts, mode, micro_batch_size, apply_chat_template, prompt_token_ids, kwargs) -> RolloutOutput:
        if kwargs:
            raise ValueError(f"generation on other ranks takes no extra arguments, got {sorted(kwargs)}")
        items = self._generate_items(prompts, mode, micro_batch_size, apply_chat_template, prompt_token_ids)
        pf = self._prefetch
        if pf is not None and pf["items"] == items:
            self.generate_finish()
            rows, self._prefetch = pf["rows"], None
        else:
            self.generate_finish()
            with self._span("rollout"):
                rows = self.exchange.call(Role.ROLLOUT, "generate", items)
        return self._merge_output(rows)

    def _serve_ref_logps(self, items: list) -> list:
        """Reference ranks: log-probs of the rows other ranks sent (grouped by the settings they share)."""
        dev = next(self.reference.parameters()).device
        out: list = [None] * len(items)
        groups: dict = {}
        for i, it in enumerate(items):
            groups.setdefault((it["pad"], it["eos"], it["mb"], tuple(sorted(it["kw"].items())), len(it["p"]), len(it["c"])),
                              []).append(i)
        chunk = self.cluster_config.training_config.compute_logps_chunk_size
        for (pad, eos, mb, kw, _, _), idx in groups.items():
            p = torch.as_tensor(np.stack([items[i]["p"] for i in idx]), device=dev)
            c = torch.as_tensor(np.stack([items[i]["c"] for i in idx]), device=dev)
            m = None if items[idx[0]]["m"] is None else torch.as_tensor(np.stack([items[i]["m"] for i in idx]), device=dev)
            fn = lambda pp, cc, mm: self.inference_worker.get_ref_per_token_logps(  # noqa: E731
                pp, cc, pad, eos, completion_mask=mm, chunk_size=chunk, **dict(kw))
            with self._span("refer_inference"):
                res = self._mb_apply(fn, (p, c, m), mb).float().cpu().numpy()
            for i, row in zip(idx, res):
                out[i] = row
        return out

    def serve(self) -> int:
        """Ranks that host no part of the training loop: answer rounds until the controllers close the cluster."""
        return self.exchange.serve()

    # ---------------------------------------------------------------- logps
    def _mb_apply(self, fn: Callable, tensors: tuple, micro_batch_size: Optional[int]):
        n = tensors[0].shape[0]
        mb = micro_batch_size or n
        outs = [fn(*[t[s0:s0 + mb] if t is not None else None for t in tensors]) for s0 in range(0, n, mb)]
        return torch.cat(outs, 0)

    def get_ref_per_token_logps(self, prompt_tokens, completion_tokens, pad_id, eos_id, micro_batch_size=None,
                                completion_mask=None, **kw):
        chunk = self.cluster_config.training_config.compute_logps_chunk_size
        if not self._ref_shares_backbone and not self.exchange.is_local(Role.REFERENCE):
            with self._span("refer_inference"):
                host = lambda t: None if t is None else t.detach().cpu().numpy()  # noqa: E731
                P, C, M = host(prompt_tokens), host(completion_tokens), host(completion_mask)
                items = [{"p": P[i], "c": C[i], "m": None if M is None else M[i], "pad": pad_id, "eos": eos_id,
                          "mb": micro_batch_size, "kw": {k: v for k, v in kw.items() if v is not None}}
                         for i in range(P.shape[0])]
                rows = self.exchange.call(Role.REFERENCE, "ref_logps", items)
                return torch.as_tensor(np.stack(rows), device=prompt_tokens.device)
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
        """Log-probs under the rollout policy's weights (the sampler's model). With the sampler on other ranks the
        actor's own weights stand in: they are what the sampler received at the last sync."""
        if self.rollout is None or not self.exchange.is_local(Role.ROLLOUT):
            return self.get_actor_per_token_logps(prompt_tokens, completion_tokens, self.tokenizer.pad_id(),
                                                  self.tokenizer.eos_id(), micro_batch_size, completion_mask, **kw)
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
        """Controllers: bring the sampler's weights up to date with the actor's; bump the global step. Ranks in
        `serve()` join the transfer when it crosses ranks."""
        self.generate_finish()
        # `free_kv_during_sync`: the paged engine gives its KV pool back for the time of the transfer (staging buffers
        # of the transfer then fit where the pool was) and allocates it again afterwards
        engine = getattr(self.rollout, "_engine", None)
        free_kv = engine is not None and bool(getattr(self._rollout_config(), "free_kv_during_sync", False))
        with self._span("weight_sync"):
            if free_kv:
                engine.delete_cache()
            try:
                if not self._rollout_shares_weights:
                    self.exchange.sync()
            finally:
                if free_kv:
                    engine.reinitialize_cache()
            if self.cluster_config.gc_collect_after_weight_sync:
                gc.collect()
        self.global_steps += 1

    def _transfer_weights(self) -> None:
        """Every rank that takes part: actor ranks offer, rollout ranks pull (`rl/reshard.py`). With adapters on
        both sides only the adapters travel; an adapter-free sampler receives `W + scale * B A`."""
        pl = self.placement
        if pl.world == 1 or (pl.same(Role.ROLLOUT, Role.ACTOR) and not self._needs_plan()):
            # same process, same layout: a device copy per tensor
            t0 = time.perf_counter()
            wait = getattr(getattr(self.actor_trainer, "optimizer", None), "wait_params", None)
            if wait is not None:
                wait()
            if self._lora and is_lora_enabled(self.rollout_actor):
                src = lora_state_dict(self.train_actor)
            else:
                from .reshard import model_sources
                src = model_sources(self.train_actor, merge_lora=self._lora)
            self.rollout.update_params(src)
            self.last_weight_sync_bytes = sum(t.numel() * t.element_size() for t in src.values())
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self.last_weight_sync_seconds = time.perf_counter() - t0
            return
        from .reshard import WeightReshard, model_sources
        t0 = time.perf_counter()
        src, dst = {}, {}
        sampler_lora = self._rollout_has_adapters()          # collective on its first call: every rank makes it
        if self.train_actor is not None:
            wait = getattr(getattr(self.actor_trainer, "optimizer", None), "wait_params", None)
            if wait is not None:
                wait()
            src = lora_state_dict(self.train_actor) if (self._lora and sampler_lora) else \
                model_sources(self.train_actor, merge_lora=self._lora)
        if self.rollout_actor is not None and self.rollout_actor is not self.train_actor:
            dst = {n: p for n, p in self.rollout_actor.named_parameters() if not sampler_lora or "lora_" in n}
        if self._resharder is None or self._resharder_key != (tuple(src), tuple(dst)):
            # the plan (who pulls which rectangle from whom) is built once; sources are re-read on every run
            self._resharder = WeightReshard(src, dst, key_map=self._tied_head_map())
            self._resharder_key = (tuple(src), tuple(dst))
        else:
            self._resharder.src = dict(src)
        self._resharder.run()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.last_weight_sync_bytes = self._resharder.bytes_pulled
        self.last_weight_sync_seconds = time.perf_counter() - t0

    def _needs_plan(self) -> bool:
        """Same ranks but different layouts (a sliced actor feeding a whole sampler) need the rectangle plan."""
        a, r = self.train_actor, self.rollout_actor
        return any(getattr(p, "shard_spec", None) is not None for m in (a, r) if m is not None for p in m.parameters())

    def _rollout_has_adapters(self) -> bool:
        flag = getattr(self, "_rollout_lora", None)
        if flag is None:
            mine = self.rollout_actor is not None and is_lora_enabled(self.rollout_actor)
            flag = mine
            pl = self.placement
            if pl.world > 1 and not pl.same(Role.ROLLOUT, Role.ACTOR):
                import torch.distributed as dist
                box = [None] * pl.world
                dist.all_gather_object(box, bool(mine) if self.rollout_actor is not None else None, group=pl.host_group)
                flag = any(b for b in box if b is not None)
            self._rollout_lora = flag
        return flag

    def _tied_head_map(self):
        return None

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
        if self.is_controller:
            self.generate_finish()
            self.exchange.stop()
        if self.actor_trainer is None:
            return
        self.actor_trainer.close()
        if self.critic_trainer is not None:
            self.critic_trainer.close()


RLEngine = RLCluster
