"""tunix_b200: a Blackwell (sm_100a) native LLM post-training framework.

Flat re-exports of the public API (the list tunix/__init__.py offers). Everything is imported lazily so that
`import tunix_b200` stays cheap and does not build or load the native libraries."""
__version__ = "0.1.0"

_EXPORTS = {
    # trainers
    "PeftTrainer": "sft.peft_trainer", "TrainingInput": "sft.peft_trainer", "TrainingConfig": "common.configs",
    "DPOTrainer": "sft.dpo.dpo_trainer", "DPOTrainingConfig": "sft.dpo.dpo_trainer", "ORPOTrainer": "sft.dpo.dpo_trainer",
    "DistillationTrainer": "distillation.distillation_trainer", "CheckpointManager": "sft.checkpoint_manager",
    "MetricsLogger": "sft.metrics_logger", "MetricsLoggerOptions": "sft.metrics_logger",
    # RL
    "RLCluster": "rl.rl_cluster", "RLEngine": "rl.rl_cluster", "ClusterConfig": "common.configs",
    "RLTrainingConfig": "common.configs", "RolloutConfig": "common.configs", "GRPOLearner": "rl.grpo.grpo_learner",
    "GRPOConfig": "rl.algorithm_config", "DAPOLearner": "rl.grpo.grpo_learner", "DrGRPOLearner": "rl.grpo.grpo_learner",
    "PPOLearner": "rl.ppo.ppo_learner", "PPOConfig": "rl.algorithm_config",
    "AgenticGRPOLearner": "rl.agentic.agentic_grpo_learner",
    # generation and models
    "Sampler": "generate.sampler", "PagedEngine": "generate.engine", "EngineServer": "generate.engine", "OpenAIServer": "generate.openai_server",
    "CacheConfig": "common.configs", "Gemma4Config": "models.gemma4", "Gemma4Multimodal": "models.gemma4_vision",
    "TokenizerAdapter": "generate.tokenizer_adapter", "AutoModel": "models.automodel", "ModelConfig": "models.config",
    "Transformer": "models.transformer", "create_model": "models.transformer",
    # adapters and optimisation
    "LoraProvider": "lora", "apply_lora_to_model": "lora", "AdamW": "optim", "SGD": "optim", "create_optimizer": "optim",
    "ShardedAdamW": "parallel.fsdp",
    # enums
    "Mode": "common.datatypes", "Role": "common.datatypes",
}

__all__ = sorted(_EXPORTS) + ["__version__"]


def __getattr__(name):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module 'tunix_b200' has no attribute {name!r}")
    import importlib
    value = getattr(importlib.import_module(f"{__name__}.{mod}"), name)
    globals()[name] = value
    return value


def __dir__():
    return __all__
