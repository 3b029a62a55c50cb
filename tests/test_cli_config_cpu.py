"""Configuration parsing in depth (test model: tests/cli/config_test.py): value typing of overrides, nested and new
keys, override files, role inheritance without shared containers, validation, optimizer / schedule factory, reward
function loading by every accepted spelling."""
import os
import textwrap

import pytest

from tunix_b200.cli import config as C

BASE = os.path.join(os.path.dirname(C.__file__), "base_config.yaml")


def _hp(*over, env=None):
    return C.HyperParameters(["prog", BASE, *over], env=env or {})


def test_override_values_are_typed_like_yaml():
    hp = _hp("batch_size=32", "optimizer_config.learning_rate=3e-4", "model_config.use_flash_attention=false",
             "model_config.model_name=qwen3-8b", "training_config.data_sharding_axis=[fsdp, tp]",
             "model_config.lora_config={rank: 8, alpha: 16.0, module_path: '.*q_proj'}", "training_config.max_steps=null")
    assert hp["batch_size"] == 32 and hp["optimizer_config"]["learning_rate"] == pytest.approx(3e-4)
    assert hp["model_config"]["use_flash_attention"] is False and hp["model_config"]["model_name"] == "qwen3-8b"
    assert hp["training_config"]["data_sharding_axis"] == ["fsdp", "tp"] and hp["training_config"]["max_steps"] is None
    assert hp["model_config"]["lora_config"] == {"rank": 8, "alpha": 16.0, "module_path": ".*q_proj"}
    assert _hp("optimizer_config.learning_rate=1")["optimizer_config"]["learning_rate"] == 1          # an int where a float is expected
    for bad in ("batch_size=1.5", "model_config.use_flash_attention=1", "batch_size=true", "model_config.model_name=3"):
        with pytest.raises(TypeError):
            _hp(bad)
    with pytest.raises(KeyError):
        _hp("nonexistent_section.key=1")
    assert _hp("model_config.config_overrides.num_layers=2")["model_config"]["config_overrides"] == {"num_layers": 2}   # new nested key


def test_roles_inherit_model_config_without_sharing_containers():
    hp = _hp("model_config.lora_config.rank=4", "actor_model_config.lora_config.rank=16", "model_config.dtype=float32")
    assert hp["model_config"]["lora_config"] == {"rank": 4}
    assert hp["actor_model_config"]["lora_config"] == {"rank": 16}                 # the role's own override wins
    assert hp["reference_model_config"]["lora_config"] == {"rank": 4} and hp["reference_model_config"]["dtype"] == "float32"
    hp.config["reference_model_config"]["lora_config"]["rank"] = 99                 # no aliasing between sections
    assert hp["model_config"]["lora_config"]["rank"] == 4 and hp["rollout_model_config"]["lora_config"]["rank"] == 4
    assert hp["reference_model_config"]["mesh"] is None and hp["critic_model_config"] is None


def test_env_overrides_and_override_files(tmp_path):
    hp = _hp(env={"T_BATCH_SIZE": "12", "T_DATA_SOURCE": "jsonl", "UNRELATED": "x", "T_NOT_A_KEY": "1"})
    assert hp["batch_size"] == 12 and hp["data_source"] == "jsonl"
    f = tmp_path / "o.yaml"
    f.write_text(textwrap.dedent("""
        batch_size: 2
        rollout_engine: paged
        training_config:
          max_steps: 7
          checkpointing_options: {max_to_keep: 5}
    """))
    hp = _hp(f"override_config_file={f}", "training_config.max_steps=9")
    assert hp["batch_size"] == 2 and hp["rollout_engine"] == "paged" and hp["training_config"]["max_steps"] == 9
    assert hp["training_config"]["checkpointing_options"]["max_to_keep"] == 5
    assert hp["training_config"]["checkpointing_options"]["save_interval_steps"] == 180      # merged, not replaced
    assert hp["rl_training_config"]["max_steps"] == 10                                        # another section keeps its own


def test_validation_messages():
    with pytest.raises(ValueError, match="batch_size must be positive"):
        _hp("batch_size=0")
    with pytest.raises(ValueError, match="rollout_engine must be"):
        _hp("rollout_engine=vllm")
    with pytest.raises(ValueError, match="differ in length"):
        _hp("model_config.mesh.shape=(2,2)", "model_config.mesh.axis_names=('fsdp',)")
    assert _hp().create_mesh() is None                                              # no process group: nothing to build


def test_optimizer_and_schedule_factory():
    hp = _hp("optimizer_config.schedule_type=warmup_cosine_decay_schedule", "optimizer_config.peak_value=1e-3",
             "optimizer_config.warmup_steps=4", "optimizer_config.decay_steps=20", "optimizer_config.end_value=1e-5")
    opt = hp.create_optimizer()
    lrs = [opt.learning_rate_at(s) for s in (0, 2, 4, 12, 20, 50)]
    assert lrs[0] == 0.0 and lrs[1] == pytest.approx(5e-4) and lrs[2] == pytest.approx(1e-3) and lrs[2] > lrs[3] > lrs[4]
    assert lrs[4] == pytest.approx(1e-5) and lrs[5] == pytest.approx(1e-5)
    const = C.create_optimizer({"opt_type": "adamw", "learning_rate": 2e-5, "weight_decay": 0.0, "b2": 0.95})
    assert const.learning_rate_at(0) == const.learning_rate_at(1000) == 2e-5
    ratio = C.create_optimizer({"schedule_type": "warmup_cosine_decay_schedule", "peak_value": 1.0, "init_value": 0.0, "end_value": 0.0,
                                "warmup_ratio": 0.25}, max_steps=40)
    assert ratio.learning_rate_at(10) == pytest.approx(1.0) and ratio.learning_rate_at(5) == pytest.approx(0.5)   # 25 % of 40 steps
    sgd = C.create_optimizer({"opt_type": "sgd", "learning_rate": 0.1, "momentum": 0.9})
    assert type(sgd).__name__.lower().startswith("sgd")
    actor = hp.create_optimizer("actor_optimizer_config", parent="rl_training_config")
    assert actor.max_grad_norm == 0.1


def test_reward_functions_load_by_every_spelling(tmp_path):
    f = tmp_path / "my_rewards.py"
    f.write_text(textwrap.dedent("""
        def helper(x):
            return x
        def length_reward(prompts, completions, **kw):
            return [float(len(c)) for c in completions]
        def other_reward(prompts, completions, **kw):
            return [0.0 for _ in completions]
        def _private_reward(*a, **k):
            return []
    """))
    assert C.load_reward_fn(str(f))(prompts=["p"], completions=["abc"]) == [3.0]          # first public *reward* function
    assert C.load_reward_fn(f"{f}:other_reward")(prompts=["p"], completions=["abc"]) == [0.0]
    assert C.load_reward_fn("tunix_b200.cli.reward_fn.gsm8k:reward_fn" if hasattr(__import__("tunix_b200.cli.reward_fn.gsm8k", fromlist=["x"]), "reward_fn")
                            else "tunix_b200.utils.math_rewards:math_reward").__name__ in ("reward_fn", "math_reward")
    assert C.load_reward_fn("tunix_b200.utils.math_rewards.format_reward").__name__ == "format_reward"
    assert C.load_reward_fn("tunix_b200/cli/reward_fn/gsm8k.py") is not None               # relative to the repository root
    empty = tmp_path / "none.py"
    empty.write_text("def helper():\n    return 1\n")
    with pytest.raises(ValueError, match="no reward function found"):
        C.load_reward_fn(str(empty))
    hp = _hp(f"reward_functions=['{f}:length_reward', 'tunix_b200.utils.math_rewards:format_reward']")
    assert [fn.__name__ for fn in hp.obtain_reward_fns()] == ["length_reward", "format_reward"]


def test_scientific_notation_without_a_dot_is_a_number(tmp_path):
    assert _hp("optimizer_config.learning_rate=3e-4")["optimizer_config"]["learning_rate"] == pytest.approx(3e-4)
    assert _hp("optimizer_config.learning_rate=1E-5")["optimizer_config"]["learning_rate"] == pytest.approx(1e-5)
    f = tmp_path / "o.yaml"
    f.write_text("optimizer_config:\n  peak_value: 2e-5\n  learning_rate: 5e-6\n")
    hp = _hp(f"override_config_file={f}")
    assert hp["optimizer_config"]["peak_value"] == pytest.approx(2e-5) and isinstance(hp["optimizer_config"]["learning_rate"], float)
    assert _hp("model_config.model_name=1e5x")["model_config"]["model_name"] == "1e5x"      # only whole numbers are converted
