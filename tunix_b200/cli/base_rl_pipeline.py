"""What the RL entry points share: role -> mesh resolution, rollout / cluster / training configs, engine
construction on the ranks that host each role, `max_steps` derivation (tunix/cli/base_rl_pipeline.py:47-899).

Mesh ownership (:135-270 there). The actor always owns a mesh (`actor_model_config.mesh`). Any other role
section that carries a `mesh` of its own gets its own ranks, carved out of the job after the actor's in the order
critic, reference, reward, rollout; a section with `mesh: null` lives on the actor's ranks, or on those of the role
named by `same_mesh_as` (chains are followed, cycles refused, a section may not have both). Equal rank sets are the
colocated layout; different ones the disaggregated layouts of `rl/placement.py`.

One process per GPU: every rank runs the same entry point; ranks that host no part of the training loop end up in
`RLCluster.serve()`.
"""
from __future__ import annotations

import ast
import dataclasses
from typing import Any, Optional

import numpy as np
import torch

from ..common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
from ..common.datatypes import Role
from ..parallel import mesh as mesh_lib
from ..rl.placement import RolePlacement
from ..rl.rl_cluster import RLCluster
from . import config as config_lib
from .peft_main import init_distributed, training_config_from
from .utils import data as data_lib, model as model_lib

ROLE_TO_MODEL_KEY = {Role.ACTOR: "actor_model_config", Role.CRITIC: "critic_model_config",
                     Role.REFERENCE: "reference_model_config", Role.REWARD: "reward_model_config",
                     Role.ROLLOUT: "rollout_model_config"}


class BasePipeline(config_lib.HyperParameters):
    default_training_mode = "grpo"

    # ------------------------------------------------------------------------------------------ meshes
    def _section(self, role: Role) -> dict:
        sec = self.config.get(ROLE_TO_MODEL_KEY[role])
        return sec if isinstance(sec, dict) else {}

    def _is_role_active(self, role: Role) -> bool:
        if role in (Role.ACTOR, Role.REFERENCE, Role.ROLLOUT):
            return True
        return bool(self.config.get(ROLE_TO_MODEL_KEY[role])) or (role == Role.CRITIC and getattr(self, "need_critic", False))

    def _same_mesh_as(self) -> dict:
        out = {}
        for role in ROLE_TO_MODEL_KEY:
            target = self._section(role).get("same_mesh_as")
            if target is None:
                continue
            if not isinstance(target, str):
                raise TypeError(f"{ROLE_TO_MODEL_KEY[role]}.same_mesh_as must be a role name, got {type(target).__name__}")
            name = target.strip().lower()
            if name not in {r.value for r in Role}:
                raise ValueError(f"unknown role name {target!r}; expected one of {sorted(r.value for r in Role)}")
            if role == Role.ACTOR:
                raise ValueError("the actor must own its mesh")
            out[role] = Role(name)
        return out

    def parse_mesh_config(self, role: Role) -> tuple:
        m = self._section(role).get("mesh") or self.config["model_config"]["mesh"]
        shape = ast.literal_eval(m["shape"]) if isinstance(m["shape"], str) else m["shape"]
        names = ast.literal_eval(m["axis_names"]) if isinstance(m["axis_names"], str) else m["axis_names"]
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        if len(shape) != len(names):
            raise ValueError(f"{ROLE_TO_MODEL_KEY[role]}.mesh: shape {shape} and axis names {tuple(names)} differ in length")
        return shape, tuple(names)

    def resolve_mesh_owners(self) -> dict:
        """role -> the role whose ranks it lives on."""
        same = self._same_mesh_as()
        base = {}
        for role in ROLE_TO_MODEL_KEY:
            if not self._is_role_active(role) and role not in same:
                continue
            has_mesh = role == Role.ACTOR or bool(self._section(role).get("mesh"))
            if has_mesh and role in same:
                raise ValueError(f"{ROLE_TO_MODEL_KEY[role]}.mesh is given, so the role owns its ranks and cannot also "
                                 "use same_mesh_as")
            base[role] = role if has_mesh else Role.ACTOR

        def owner_of(role: Role, seen: set) -> Role:
            if role in seen:
                raise ValueError("same_mesh_as contains a cycle")
            if role not in same:
                return base[role]
            seen.add(role)
            if same[role] not in base:
                raise ValueError(f"role {same[role].value!r} is not active in this config")
            return owner_of(same[role], seen)
        return {role: owner_of(role, set()) for role in base}

    def create_role_to_mesh(self, world: Optional[int] = None) -> dict:
        """role -> `parallel.mesh.Mesh`. Owners get disjoint rank ranges in role order; the actor's default mesh
        `(1,)` stretches over whatever the other owners leave."""
        import torch.distributed as dist
        world = world if world is not None else (dist.get_world_size() if dist.is_initialized() else 1)
        owners = self.resolve_mesh_owners()
        order = [r for r in ROLE_TO_MODEL_KEY if r in set(owners.values())]
        policies = {(self._section(r).get("mesh") or {}).get("allocation_policy", "COMPACT") for r in order}
        if len(policies) > 1:
            raise ValueError(f"all owned meshes must use one mesh.allocation_policy, got {sorted(policies)}")
        shapes = {r: self.parse_mesh_config(r) for r in order}
        others = sum(int(np.prod(shapes[r][0])) for r in order if r != Role.ACTOR)
        a_shape, a_names = shapes[Role.ACTOR]
        if int(np.prod(a_shape)) == 1 and len(a_shape) == 1 and world - others > 1:
            shapes[Role.ACTOR] = ((world - others,), a_names)
        slices = mesh_lib.allocate_named_mesh_device_slices({r.value: int(np.prod(shapes[r][0])) for r in order},
                                                            num_devices=world, allocation_policy=policies.pop())
        built = {r: mesh_lib.create_mesh(shapes[r][0], shapes[r][1], ranks=slices[r.value], set_current=False)
                 for r in order}
        return {role: built[owner] for role, owner in owners.items()}

    # ----------------------------------------------------------------------------------------- configs
    def create_rollout_config(self) -> RolloutConfig:
        """`rollout_config` fields pass through; kv_cache_size defaults to prompt + generation + 256 and the number
        of running requests to batch_size x num_generations (agentic: `max_concurrency`), as in the reference
        (:272-426)."""
        rc = dict(self.config["rollout_config"])
        valid = {f.name for f in dataclasses.fields(RolloutConfig)}
        kw = {k: v for k, v in rc.items() if k in valid and v is not None}
        if "total_generation_steps" in rc:
            kw["max_tokens_to_generate"] = rc["total_generation_steps"]
        mp, mg = rc.get("max_prompt_length", 0), rc.get("total_generation_steps", 0)
        kw["kv_cache_size"] = rc.get("kv_cache_size") or (mp + mg + 256)
        mode = self.config.get("training_mode") or self.default_training_mode
        if mode.startswith("agentic"):
            running = int((self.config.get("agentic_config") or {}).get("max_concurrency", 16))
        else:
            algo = self.config.get(f"{mode}_config") or {}
            running = int(self.config.get("batch_size", 1)) * int(algo.get("num_generations", 1))
        kw.setdefault("max_running_requests", max(running, 1))
        return RolloutConfig(**kw)

    def create_rl_training_config(self, need_critic: bool = False) -> RLTrainingConfig:
        rt = dict(self.config["rl_training_config"])
        aoc, coc = rt.pop("actor_optimizer_config"), rt.pop("critic_optimizer_config", None)
        max_steps = rt.get("max_steps")
        return training_config_from(
            rt, RLTrainingConfig, actor_optimizer=config_lib.create_optimizer(aoc, max_steps),
            critic_optimizer=config_lib.create_optimizer(coc or aoc, max_steps) if need_critic else None)

    def create_cluster_config(self, role_to_mesh: dict, need_critic: bool = False) -> ClusterConfig:
        return ClusterConfig(role_to_mesh=role_to_mesh, rollout_engine=self.config["rollout_engine"],
                             offload_to_cpu=self.config["offload_to_cpu"],
                             training_config=self.create_rl_training_config(need_critic),
                             rollout_config=self.create_rollout_config())

    # ------------------------------------------------------------------------------------------ engine
    def create_rl_engine(self, dev=None, need_critic: bool = False) -> RLCluster:
        """Models are built only on the ranks that host their role (:514-612)."""
        import torch.distributed as dist
        from ..lora import is_lora_enabled
        self.need_critic = need_critic
        dev = dev if dev is not None else init_distributed()
        r2m = self.create_role_to_mesh() if dist.is_initialized() and dist.get_world_size() > 1 else {}
        pl = RolePlacement(r2m)
        tok = model_lib.create_tokenizer(self.config["tokenizer_config"])
        mk = lambda key: model_lib.create_model(self.config[key], device=dev)  # noqa: E731
        actor = mk("actor_model_config") if pl.has(Role.ACTOR) else None
        lora = bool(self.config["actor_model_config"].get("lora_config"))
        reference = None
        if pl.has(Role.REFERENCE) and not (lora and pl.same(Role.REFERENCE, Role.ACTOR)):
            reference = mk("reference_model_config")
            if actor is not None and not is_lora_enabled(actor):
                reference.load_state_dict(actor.state_dict())
            for p in reference.parameters():
                p.requires_grad_(False)
        rollout_model = None
        if pl.has(Role.ROLLOUT) and not pl.same(Role.ROLLOUT, Role.ACTOR):
            rollout_model = mk("rollout_model_config")
            for p in rollout_model.parameters():
                p.requires_grad_(False)
        critic = None
        if need_critic and pl.has(Role.CRITIC) and actor is not None:
            from ..rl.utils import create_critic_model
            critic = create_critic_model(actor)
        cc = self.create_cluster_config(r2m, need_critic)
        cluster = RLCluster(actor=actor, reference=reference, critic=critic, rollout_model=rollout_model, tokenizer=tok,
                            cluster_config=cc, placement=pl,
                            separate_rollout_copy=bool(self._section(Role.ROLLOUT).get("separate_copy", False)))
        if not pl.same(Role.ROLLOUT, Role.ACTOR):
            cluster.exchange.sync()      # the sampler starts from the actor's weights, whatever it was built with
        return cluster

    # ------------------------------------------------------------------------------------- step counts
    def compute_max_steps(self, dataset_length: Optional[int]) -> int:
        """max_steps from the dataset length, `num_batches`, `num_train_epochs` and `train_fraction` (:618-736)."""
        c = self.config
        rt = c["rl_training_config"]
        max_steps = rt.get("max_steps")
        if dataset_length is None and not max_steps:
            raise ValueError("max_steps must be given: the dataset length cannot be determined")
        batch_size = c.get("batch_size", 1)
        num_batches = c.get("num_batches")
        if not num_batches and not dataset_length:
            if max_steps:
                return int(max_steps)
            raise ValueError("num_batches is not given and cannot be derived: the dataset length is unknown")
        if not num_batches:
            num_batches = dataset_length // batch_size
        c["num_batches"] = num_batches
        epochs = c.get("num_train_epochs") or 1
        frac = c.get("train_fraction")
        if not frac or frac <= 0.0 or frac > 1.0:
            frac = 0.8
        allowed = int(num_batches * epochs * frac)
        if not max_steps:
            max_steps = allowed
        elif max_steps > allowed:
            raise ValueError(f"maximum allowed value for max_steps is {allowed}, but {max_steps} is specified")
        return int(max_steps)

    def compute_params(self, dataset_length: Optional[int]) -> int:
        """Writes `max_steps` back and fills the optimizers' `decay_steps` / `warmup_steps` where they are unset."""
        rt = self.config["rl_training_config"]
        max_steps = self.compute_max_steps(dataset_length)
        rt["max_steps"] = max_steps
        for key in ("actor_optimizer_config", "critic_optimizer_config"):
            opt = rt.get(key)
            if opt is None:
                continue
            if not isinstance(opt, dict):
                raise ValueError(f"rl_training_config.{key} must be a mapping")
            if not opt.get("decay_steps"):
                opt["decay_steps"] = max_steps
            if not opt.get("warmup_steps"):
                ratio = self.config.get("warmup_ratio", opt.get("warmup_ratio", 0.1))
                opt["warmup_steps"] = self.config.get("warmup_steps", ratio * max_steps)
        return max_steps

    # ------------------------------------------------------------------------------------------- data
    def prompt_dataset(self, tokenizer, vocab_size: int):
        c = self.config
        n = c["num_batches"] or (c["rl_training_config"].get("max_steps") or 10)
        if c["data_source"] == "synthetic":
            return data_lib.synthetic_prompts(c["batch_size"], min(c["rollout_config"]["max_prompt_length"], 32), vocab_size, n)
        import os
        path = os.path.join(c["data_directory"], c["dataset_name"] or "train.jsonl")
        tpl = (lambda p: tokenizer.apply_chat_template([{"role": "user", "content": p}])) \
            if c["apply_chat_template_to_dataset"] else None
        return data_lib.jsonl_prompts(path, c["batch_size"], tpl, c["num_train_epochs"])

    def run(self, build_learner, need_critic: bool = False):
        """The whole job on this rank: engine, then either the training loop (actor ranks) or `serve()`."""
        dev = init_distributed()
        cluster = self.create_rl_engine(dev, need_critic)
        if not cluster.is_controller:
            cluster.serve()
            return cluster
        learner = build_learner(cluster)
        vocab = cluster.train_actor.config.vocab_size
        learner.train(self.prompt_dataset(cluster.tokenizer, vocab))
        return cluster
