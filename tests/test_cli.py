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
