"""`python -m tunix_b200.cli.ppo_main base_config.yaml key=value ...` — PPO (tunix/cli/ppo_main.py:35-122)."""
from __future__ import annotations

import sys

from ..rl.algorithm_config import PPOConfig
from ..rl.ppo.ppo_learner import PPOLearner
from . import config as config_lib
from .grpo_main import create_rl_engine, prompt_dataset
from .peft_main import init_distributed


def main(argv=None):
    hp = config_lib.HyperParameters(sys.argv if argv is None else argv)
    dev = init_distributed()
    cluster = create_rl_engine(hp, dev, need_critic=True)
    learner = PPOLearner(cluster, PPOConfig(**hp["ppo_config"]), reward_fns=hp.obtain_reward_fns())
    learner.train(prompt_dataset(hp, cluster.tokenizer, cluster.train_actor.config.vocab_size))
    return cluster


if __name__ == "__main__":
    main()
