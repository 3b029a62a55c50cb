"""`python -m tunix_b200.cli.grpo_main base_config.yaml key=value ...` — GRPO (and DAPO / Dr.GRPO / GSPO-token via
`grpo_config`), non-agentic or agentic (`training_mode=agentic_grpo`) (tunix/cli/grpo_main.py:43-201,
tunix/cli/base_rl_pipeline.py:47-899)."""
from __future__ import annotations

import sys

from ..rl.algorithm_config import DAPOConfig, DrGRPOConfig, GRPOConfig
from ..rl.grpo.dapo_learner import DAPOLearner
from ..rl.grpo.drgrpo_learner import DrGRPOLearner
from ..rl.grpo.grpo_learner import GRPOLearner
from ..rl.rl_cluster import RLCluster
from .base_rl_pipeline import BasePipeline


def create_rl_engine(hp, dev=None, need_critic: bool = False) -> RLCluster:
    """Kept for callers that hold a `HyperParameters`: the pipeline's engine construction on the same config."""
    pipe = hp if isinstance(hp, BasePipeline) else BasePipeline.__new__(BasePipeline)
    if pipe is not hp:
        pipe.__dict__.update(hp.__dict__)
    return pipe.create_rl_engine(dev, need_critic)


def prompt_dataset(hp, tokenizer, vocab_size):
    return BasePipeline.prompt_dataset(hp, tokenizer, vocab_size)


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
    """Every rank runs this. Actor ranks train; ranks that only host the sampler or the reference serve them
    (`actor_model_config.mesh`, `rollout_model_config.mesh`, `same_mesh_as` decide who is who)."""
    hp = BasePipeline(sys.argv if argv is None else argv)

    def build(cluster):
        g = dict(hp["grpo_config"])
        variant = g.pop("algo_variant", "grpo")
        cfg_cls, learner_cls = {"dapo": (DAPOConfig, DAPOLearner), "drgrpo": (DrGRPOConfig, DrGRPOLearner)}.get(
            variant, (GRPOConfig, GRPOLearner))
        algo = cfg_cls(**g)
        rewards = hp.obtain_reward_fns()
        if hp["training_mode"] == "agentic_grpo":
            from ..rl.agentic.agentic_grpo_learner import AgenticGRPOLearner
            return AgenticGRPOLearner(cluster, rewards, algo, **agentic_kwargs(hp))
        return learner_cls(cluster, rewards, algo)
    return hp.run(build)


if __name__ == "__main__":
    main()
