"""`python -m tunix_b200.cli.ppo_main base_config.yaml key=value ...` — PPO (tunix/cli/ppo_main.py:35-122)."""
from __future__ import annotations

import sys

from ..rl.algorithm_config import PPOConfig
from ..rl.ppo.ppo_learner import PPOLearner
from .base_rl_pipeline import BasePipeline


def main(argv=None):
    hp = BasePipeline(sys.argv if argv is None else argv)
    return hp.run(lambda cluster: PPOLearner(cluster, PPOConfig(**hp["ppo_config"]), reward_fns=hp.obtain_reward_fns()),
                  need_critic=True)


if __name__ == "__main__":
    main()
