"""`python -m tunix_b200.cli.grpo_main base_config.yaml key=value ...` — GRPO (and DAPO / Dr.GRPO / GSPO-token via
`grpo_config`), non-agentic or agentic (`training_mode=agentic_grpo`) (tunix/cli/grpo_main.py:43-201,
tunix/cli/base_rl_pipeline.py:47-899)."""
from __future__ import annotations

import sys

from ..common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
from ..rl.algorithm_config import DAPOConfig, DrGRPOConfig, GRPOConfig
from ..rl.grpo.grpo_learner import DAPOLearner, DrGRPOLearner, GRPOLearner
from ..rl.rl_cluster import RLCluster
from . import config as config_lib
from .peft_main import init_distributed, training_config_from
from .utils import data as data_lib, model as model_lib


def rollout_config_from(hp) -> RolloutConfig:
    rc = hp["rollout_config"]
    return RolloutConfig(max_tokens_to_generate=rc["total_generation_steps"], max_prompt_length=rc["max_prompt_length"],
                         temperature=rc["temperature"], top_p=rc.get("top_p"), top_k=rc.get("top_k"),
                         kv_cache_size=rc["max_prompt_length"] + rc["total_generation_steps"] + 8)


def create_rl_engine(hp, dev, need_critic: bool = False) -> RLCluster:
    actor = model_lib.create_model(hp["actor_model_config"], device=dev)
    tok = model_lib.create_tokenizer(hp["tokenizer_config"])
    from ..lora import is_lora_enabled
    reference = None
    if not is_lora_enabled(actor):
        reference = model_lib.create_model(hp["reference_model_config"], device=dev)
        reference.load_state_dict(actor.state_dict())
        for p in reference.parameters():
            p.requires_grad_(False)
    critic = None
    if need_critic:
        from ..rl.utils import create_critic_model
        critic = create_critic_model(actor)
    rt = dict(hp["rl_training_config"])
    aoc, coc = rt.pop("actor_optimizer_config"), rt.pop("critic_optimizer_config", None)
    max_steps = rt.get("max_steps")
    tc = training_config_from(rt, RLTrainingConfig, actor_optimizer=config_lib.create_optimizer(aoc, max_steps),
                              critic_optimizer=config_lib.create_optimizer(coc or aoc, max_steps) if need_critic else None)
    cc = ClusterConfig(role_to_mesh={}, rollout_engine=hp["rollout_engine"], offload_to_cpu=hp["offload_to_cpu"],
                       training_config=tc, rollout_config=rollout_config_from(hp))
    return RLCluster(actor=actor, reference=reference, critic=critic, tokenizer=tok, cluster_config=cc)


def prompt_dataset(hp, tokenizer, vocab_size):
    c = hp.config
    n = c["num_batches"] or (c["rl_training_config"].get("max_steps") or 10)
    if c["data_source"] == "synthetic":
        return data_lib.synthetic_prompts(c["batch_size"], min(c["rollout_config"]["max_prompt_length"], 32), vocab_size, n)
    import os
    path = os.path.join(c["data_directory"], c["dataset_name"] or "train.jsonl")
    tpl = (lambda p: tokenizer.apply_chat_template([{"role": "user", "content": p}])) if c["apply_chat_template_to_dataset"] else None
    return data_lib.jsonl_prompts(path, c["batch_size"], tpl, c["num_train_epochs"])


def agentic_kwargs(hp) -> dict:
    """Constructor arguments of the agentic learner from the `agentic_config` section (all optional)."""
    try:
        a = dict(hp["agentic_config"] or {})
    except KeyError:
        return {}
    from ..rl.agentic.agents.model_agent import ModelAgent
    from ..rl.agentic.agents.tool_agent import ToolAgent
    from ..rl.agentic.environments.task_environment import TaskEnvironment
    from ..rl.agentic.environments.tool_environment import ToolEnvironment
    from ..rl.agentic.parser.chat_template_parser import get_parser
    from ..rl.agentic.tools.calculator_tool import CalculatorTool
    tools = {"calculator": CalculatorTool}
    chosen = [tools[t]() for t in a.get("tools", []) if t in tools]
    kw = {"max_turns": int(a.get("max_turns", 1)), "max_concurrency": int(a.get("max_concurrency", 16)),
          "off_policy_steps": int(a.get("off_policy_steps", 0)), "episode_timeout": float(a.get("episode_timeout", 600.0)),
          "chat_parser": get_parser(a.get("chat_parser", "default"))}
    if a.get("agent", "model") == "tool":
        kw["agent_class"], kw["agent_kwargs"] = ToolAgent, {"tools": {t.name: t for t in chosen}}
    elif a.get("agent") == "frozenlake":
        from ..rl.agentic.environments.frozenlake_environment import FrozenLakeAgent
        kw["agent_class"] = FrozenLakeAgent
    else:
        kw["agent_class"] = ModelAgent
    if a.get("environment") == "frozenlake":
        from ..rl.agentic.environments.frozenlake_environment import FrozenLakeEnv
        kw["env_class"], kw["env_kwargs"] = FrozenLakeEnv, {"max_steps": kw["max_turns"],
                                                            "is_slippery": bool(a.get("is_slippery", False))}
    elif a.get("environment", "task") == "tool":
        kw["env_class"], kw["env_kwargs"] = ToolEnvironment, {"tools": chosen, "reward_fn": a.get("reward_fn", "exact_match"),
                                                              "max_steps": kw["max_turns"]}
    else:
        kw["env_class"], kw["env_kwargs"] = TaskEnvironment, {"reward_fn": a.get("reward_fn", "exact_match")}
    return kw


def main(argv=None):
    hp = config_lib.HyperParameters(sys.argv if argv is None else argv)
    dev = init_distributed()
    cluster = create_rl_engine(hp, dev)
    g = dict(hp["grpo_config"])
    variant = g.pop("algo_variant", "grpo")
    cfg_cls, learner_cls = {"dapo": (DAPOConfig, DAPOLearner), "drgrpo": (DrGRPOConfig, DrGRPOLearner)}.get(
        variant, (GRPOConfig, GRPOLearner))
    algo = cfg_cls(**g)
    rewards = hp.obtain_reward_fns()
    if hp["training_mode"] == "agentic_grpo":
        from ..rl.agentic.agentic_grpo_learner import AgenticGRPOLearner
        learner = AgenticGRPOLearner(cluster, rewards, algo, **agentic_kwargs(hp))
    else:
        learner = learner_cls(cluster, rewards, algo)
    learner.train(prompt_dataset(hp, cluster.tokenizer, cluster.train_actor.config.vocab_size))
    return cluster


if __name__ == "__main__":
    main()
