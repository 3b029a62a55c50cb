"""Tag names of the second-generation tracer (tunix/perf/experimental/constants.py:17-37)."""
STEP = "global_step"
MINI_BATCH = "mini_batch"
MICRO_BATCH = "micro_batch"
ROLE = "role"
GROUP = "group"
PAIR = "pair"
POLICY_VERSION = "policy_version"

ROLLOUT, REFERENCE, ACTOR, CRITIC, REWARD, WEIGHT_SYNC, DATA = "rollout", "reference", "actor", "critic", "reward", "weight_sync", "data"

# Span names shared by the timelines of the RL loop, and the tag under which a queue span keeps the name of the span it
# waited for (tunix/perf/experimental/constants.py:24-37)
NAME = "NAME"
DATA_LOADING = "data_loading"
REFERENCE_INFERENCE = "reference_inference"
OLD_ACTOR_INFERENCE = "old_actor_inference"
ADVANTAGE_COMPUTATION = "advantage_computation"
PEFT_TRAIN = "peft_train"
ENVIRONMENT = "environment"
QUEUE = "queue"
