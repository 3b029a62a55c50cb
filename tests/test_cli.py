"""CLI config precedence / validation and end-to-end tiny runs of the three entry points."""
import os

import pytest

from tunix_b200.cli import config as C
from tunix_b200.cli import grpo_main, peft_main, ppo_main

BASE = os.path.join(os.path.dirname(C.__file__), "base_config.yaml")
TINY = ["model_config.config_overrides={num_layers: 1, vocab_size: 300, embed_dim: 32, hidden_dim: 64, num_heads: 2, head_dim: 16, num_kv_heads: 1}",
        "tokenizer_config.tokenizer_type=char", "batch_size=4", "max_target_length=16"]


def test_overrides_env_and_conflicts(tmp_path):
    hp = C.HyperParameters(["x", BASE, "batch_size=8", "training_config.max_steps=3", "optimizer_config.learning_rate=0.001"], env={})
    assert hp["batch_size"] == 8 and hp["training_config"]["max_steps"] == 3
    hp = C.HyperParameters(["x", BASE], env={"T_BATCH_SIZE": "4"})
    assert hp["batch_size"] == 4
    with pytest.raises(ValueError):
        C.HyperParameters(["x", BASE, "batch_size=8"], env={"T_BATCH_SIZE": "4"})
    with pytest.raises(TypeError):
        C.HyperParameters(["x", BASE, "batch_size=abc"], env={})
    with pytest.raises(KeyError):
        C.HyperParameters(["x", BASE, "no_such_key=1"], env={})
    over = tmp_path / "o.yaml"
    over.write_text("batch_size: 2\nmodel_config:\n  lora_config:\n    rank: 4\n")
    hp = C.HyperParameters(["x", BASE, f"override_config_file={over}", "batch_size=6"], env={})
    assert hp["batch_size"] == 6 and hp["model_config"]["lora_config"] == {"rank": 4}
    assert hp["actor_model_config"]["lora_config"] == {"rank": 4}     # roles inherit from model_config


def test_optimizer_factory_and_reward_loading():
    hp = C.HyperParameters(["x", BASE], env={})
    opt = hp.create_optimizer()
    assert abs(opt.learning_rate_at(10) - 0.0) < 1e-12 and opt.learning_rate_at(5) > 0 and opt.max_grad_norm == 0.1
    fns = hp.obtain_reward_fns()
    assert fns[0](prompts=["q"], completions=["<answer>42</answer>"], answer=["42"]) == [1.0]


def test_peft_main_runs(tmp_path):
    tr = peft_main.main(["x", BASE, *TINY, "training_config.max_steps=2", f"training_config.checkpoint_root_directory={tmp_path}/ck",
                         f"training_config.metrics_logging_options.log_dir={tmp_path}/log"])
    assert tr.train_steps == 2
    assert os.path.exists(tmp_path / "log" / "metrics.jsonl")


def test_grpo_and_ppo_main_run(tmp_path):
    common = [*TINY, "rl_training_config.max_steps=1", "rl_training_config.checkpoint_root_directory=", "rollout_config.total_generation_steps=4",
              "rollout_config.max_prompt_length=8", "rl_training_config.metrics_logging_options.log_dir=",
              "actor_model_config.config_overrides={num_layers: 1, vocab_size: 300, embed_dim: 32, hidden_dim: 64, num_heads: 2, head_dim: 16, num_kv_heads: 1}",
              "reference_model_config.config_overrides={num_layers: 1, vocab_size: 300, embed_dim: 32, hidden_dim: 64, num_heads: 2, head_dim: 16, num_kv_heads: 1}"]
    cl = grpo_main.main(["x", BASE, *common])
    assert cl.global_steps == 1
    cl = ppo_main.main(["x", BASE, *common])
    assert cl.global_steps == 1


def test_sft_loader_reads_chat_rows_with_assistant_only_loss(tmp_path):
    import json
    import numpy as np
    from tests.test_sampler_cpu import CharTok
    from tunix_b200.cli.utils.data import chat_row_tokens, jsonl_sft
    from tunix_b200.rl.agentic.parser.chat_template_parser import get_parser
    tok, parser = CharTok(), get_parser("qwen")
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "4"},
            {"role": "user", "content": "sure?"}, {"role": "assistant", "content": "yes"}]
    ids, mask = chat_row_tokens(msgs, tok, parser)
    assert ids == tok.encode(parser.parse(msgs)) and len(mask) == len(ids)
    # the loss covers exactly the assistant's words and their end markers
    want = sum(len(tok.encode(parser.render_message(m))) - len(tok.encode(parser.generation_prompt)) for m in msgs if m["role"] == "assistant")
    assert int(sum(mask)) == want and mask[0] == 0.0 and mask[-1] == 1.0
    path = tmp_path / "sft.jsonl"
    with open(path, "w") as f:
        f.write(json.dumps({"messages": msgs, "reward": 1.0}) + "\n")
        f.write(json.dumps({"text": "plain text row"}) + "\n")
    batch = next(iter(jsonl_sft(str(path), tok, 2, 256)))
    toks, m = np.asarray(batch.input_tokens), np.asarray(batch.input_mask)
    assert toks.shape == (2, 256) and m[0].sum() == want and toks[0, :len(ids)].tolist() == ids
    assert m[1].sum() == len("plain text row") + 1


def test_role_to_mesh_resolution_and_step_derivation():
    """Which role lives on whose ranks, from `mesh` / `same_mesh_as` in the role sections; max_steps from the data."""
    from tunix_b200.cli.base_rl_pipeline import BasePipeline
    from tunix_b200.common.datatypes import Role
    from tunix_b200.rl.placement import RolePlacement
    # default: everything on the actor's ranks, whose "(1,)" mesh stretches over the job
    hp = BasePipeline(["x", BASE], env={})
    r2m = hp.create_role_to_mesh(world=8)
    pl = RolePlacement(r2m, world=8, rank=0, make_groups=False)
    assert pl.layout == "colocated" and pl.ranks(Role.ROLLOUT) == list(range(8)) and pl.axis_size(Role.ACTOR, "fsdp") == 8
    # the sampler on 4 ranks of its own, the reference with it; the actor keeps the rest as (2, 2) fsdp x tp
    hp = BasePipeline(["x", BASE, "actor_model_config.mesh.shape=(2,2)", "actor_model_config.mesh.axis_names=('fsdp','tp')",
                       "rollout_model_config.mesh={shape: '(4,)', axis_names: \"('fsdp',)\", allocation_policy: COMPACT}",
                       "reference_model_config.same_mesh_as=rollout"], env={})
    r2m = hp.create_role_to_mesh(world=8)
    pl = RolePlacement(r2m, world=8, rank=5, make_groups=False)
    assert pl.ranks(Role.ACTOR) == [0, 1, 2, 3] and pl.ranks(Role.ROLLOUT) == pl.ranks(Role.REFERENCE) == [4, 5, 6, 7]
    assert pl.layout == "disaggregated" and not pl.is_controller and pl.axis_size(Role.ACTOR, "tp") == 2
    with pytest.raises(ValueError, match="cycle"):
        BasePipeline(["x", BASE, "reference_model_config.same_mesh_as=rollout", "rollout_model_config.same_mesh_as=reference"],
                     env={}).create_role_to_mesh(world=4)
    with pytest.raises(ValueError, match="cannot also"):
        BasePipeline(["x", BASE, "rollout_model_config.mesh={shape: '(2,)', axis_names: \"('fsdp',)\"}",
                      "rollout_model_config.same_mesh_as=actor"], env={}).create_role_to_mesh(world=4)
    with pytest.raises(ValueError, match="cannot allocate"):
        BasePipeline(["x", BASE, "actor_model_config.mesh.shape=(4,)",
                      "rollout_model_config.mesh={shape: '(4,)', axis_names: \"('fsdp',)\"}"], env={}).create_role_to_mesh(world=6)
    # steps: 100 rows / batch 16 = 6 batches, 2 epochs, 80 % for training -> 9 steps; schedules follow
    hp = BasePipeline(["x", BASE, "rl_training_config.max_steps=0", "num_train_epochs=2", "train_fraction=0.8",
                       "rl_training_config.actor_optimizer_config.decay_steps=0",
                       "rl_training_config.actor_optimizer_config.warmup_steps=0"], env={})
    assert hp.compute_params(100) == 9
    aoc = hp["rl_training_config"]["actor_optimizer_config"]
    assert hp["rl_training_config"]["max_steps"] == 9 and aoc["decay_steps"] == 9 and abs(aoc["warmup_steps"] - 0.9) < 1e-9
    hp = BasePipeline(["x", BASE, "rl_training_config.max_steps=50"], env={})
    with pytest.raises(ValueError, match="maximum allowed"):
        hp.compute_max_steps(100)
    rc = BasePipeline(["x", BASE, "batch_size=8", "grpo_config.num_generations=4"], env={}).create_rollout_config()
    assert rc.kv_cache_size == 256 + 768 + 256 and rc.max_running_requests == 32 and rc.max_tokens_to_generate == 768


def _cli_rank(rank, world, port, out):
    import sys
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    tiny = "{num_layers: 1, vocab_size: 300, embed_dim: 32, hidden_dim: 64, num_heads: 2, head_dim: 16, num_kv_heads: 1}"
    argv = ["x", BASE, "tokenizer_config.tokenizer_type=char", "batch_size=2", "rl_training_config.max_steps=2",
            "rl_training_config.checkpoint_root_directory=", "rl_training_config.metrics_logging_options.log_dir=",
            "rollout_config.total_generation_steps=4", "rollout_config.max_prompt_length=8",
            f"actor_model_config.config_overrides={tiny}", f"reference_model_config.config_overrides={tiny}",
            f"rollout_model_config.config_overrides={tiny}", "rollout_model_config.rng_seed=9",
            "actor_model_config.mesh.shape=(2,)",
            "rollout_model_config.mesh={shape: '(1,)', axis_names: \"('fsdp',)\", allocation_policy: COMPACT}"]
    cl = grpo_main.main(argv)
    import torch
    torch.save({"controller": cl.is_controller, "steps": cl.global_steps,
                "w": torch.cat([p.detach().reshape(-1) for p in (cl.train_actor or cl.rollout_actor).parameters()])},
               f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_grpo_main_on_three_ranks_with_the_sampler_on_its_own_rank(tmp_path):
    """`torchrun`-style launch of the entry point on gloo ranks: ranks 0-1 train (sharded optimizer), rank 2 serves the
    sampler, whose weights (built from another seed) follow the actor's."""
    import torch
    import torch.multiprocessing as mp
    out = str(tmp_path / "r")
    mp.spawn(_cli_rank, args=(3, 29761, out), nprocs=3, join=True)
    res = [torch.load(f"{out}.{r}") for r in range(3)]
    assert [r["controller"] for r in res] == [True, True, False] and res[0]["steps"] == 2
    assert torch.equal(res[0]["w"], res[1]["w"]) and torch.allclose(res[2]["w"], res[0]["w"], atol=1e-6)
