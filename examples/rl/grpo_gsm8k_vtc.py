"""GRPO on grade-school math with the VTC recipe, as a script (the job of examples/math_gsm8k/qwen3_grpo_demo.py).

    PYTHONPATH=. python examples/rl/grpo_gsm8k_vtc.py --data /data/gsm8k --model-path /ckpt/Qwen3-1.7B --model qwen3-1.7b
    PYTHONPATH=. python examples/rl/grpo_gsm8k_vtc.py --tiny --steps 2            # random toy model, built-in sample data, CPU

`--data` is a directory (or file) of `{"question", "answer"}` records, the answer ending in `#### <number>` as in GSM8K
(`.jsonl`, `.json` or `.parquet`; nothing is downloaded). The prompt opens the `<reasoning>` block for the model
(`utils/gsm8k_vtc.py`), the reward is graded (1.0 format + answer, 0.5 answer only, 0.1 format only), the solve-rate
metrics of every group are logged beside the learner's own."""
import argparse
import json
import os
import tempfile

import torch

from tunix_b200 import optim
from tunix_b200.common.configs import ClusterConfig, MetricsLoggerOptions, RLTrainingConfig, RolloutConfig
from tunix_b200.lora import LoraProvider, apply_lora_to_model
from tunix_b200.rl.algorithm_config import GRPOConfig
from tunix_b200.rl.grpo.grpo_learner import GRPOLearner
from tunix_b200.rl.rl_cluster import RLCluster
from tunix_b200.utils import gsm8k_vtc, script_utils

_SAMPLE = [("Tom has 3 apples and buys 4 more. How many apples does he have?", "3 + 4 = 7 #### 7"),
           ("A book costs 12 dollars. How much do 5 books cost?", "12 * 5 = 60 #### 60"),
           ("There are 20 birds; 8 fly away. How many are left?", "20 - 8 = 12 #### 12"),
           ("Each box holds 6 eggs. How many eggs are in 7 boxes?", "6 * 7 = 42 #### 42")]


def build_model(a, device):
    if a.tiny:
        from tunix_b200.experimental.worker.factories import ByteTokenizer, toy_config
        from tunix_b200.models.transformer import create_model
        return create_model(toy_config().replace(max_position=2048), device=device, seed=0), ByteTokenizer()
    from tunix_b200.generate.tokenizer_adapter import Tokenizer
    from tunix_b200.models.automodel import AutoModel, ModelSource
    model, path = AutoModel.from_pretrained(a.model, model_source=ModelSource.LOCAL, model_path=a.model_path, device=device)
    return model, Tokenizer("huggingface", path)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--data", default=None)
    ap.add_argument("--model", default="qwen3-1.7b")
    ap.add_argument("--model-path", default=None)
    ap.add_argument("--tiny", action="store_true", help="random toy model, byte tokenizer and four built-in problems")
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--batch-size", type=int, default=8, help="prompts per step")
    ap.add_argument("--generations", type=int, default=8)
    ap.add_argument("--max-new-tokens", type=int, default=512)
    ap.add_argument("--lora-rank", type=int, default=0)
    ap.add_argument("--lr", type=float, default=1e-6)
    ap.add_argument("--engine", default=None, help="vanilla | paged (default: paged on a GPU)")
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--checkpoint-dir", default=None)
    a = ap.parse_args(argv)
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    if a.tiny:
        a.batch_size, a.generations, a.max_new_tokens = min(a.batch_size, 2), min(a.generations, 2), min(a.max_new_tokens, 16)
    tmp = None
    if a.data is None:
        tmp = tempfile.TemporaryDirectory()
        a.data = os.path.join(tmp.name, "train.jsonl")
        with open(a.data, "w") as f:
            for q, ans in _SAMPLE * 4:
                f.write(json.dumps({"question": q, "answer": ans}) + "\n")
    train, _ = script_utils.get_train_and_eval_datasets(a.data, "train", seed=0, system_prompt="", batch_size=a.batch_size,
                                                        num_batches=a.steps, train_fraction=1.0, num_epochs=None,
                                                        answer_extractor=gsm8k_vtc.extract_hash_answer)
    for b in train:                                   # the recipe's prompt, fed verbatim (no chat template)
        b["prompts"] = [gsm8k_vtc.build_prompt(q) for q in b["question"]]
    model, tok = build_model(a, device)
    if a.lora_rank:
        apply_lora_to_model(model, LoraProvider(module_path=r".*(q_proj|k_proj|v_proj|o_proj|gate_proj|up_proj|down_proj)",
                                                rank=a.lora_rank, alpha=2.0 * a.lora_rank))
    prompt_len = 1 << (max(len(tok.encode(p)) for b in train for p in b["prompts"]) - 1).bit_length()
    cluster = RLCluster(actor=model, tokenizer=tok, cluster_config=ClusterConfig(
        role_to_mesh={}, rollout_engine=a.engine or ("paged" if device.type == "cuda" and not a.tiny else "vanilla"),
        training_config=RLTrainingConfig(eval_every_n_steps=10 ** 9, max_steps=a.steps, actor_optimizer=optim.AdamW(a.lr, max_grad_norm=1.0),
                                         mini_batch_size=a.batch_size, train_micro_batch_size=max(a.batch_size // 4, 1),
                                         checkpoint_root_directory=a.checkpoint_dir,
                                         metrics_logging_options=MetricsLoggerOptions(log_dir=a.log_dir) if a.log_dir else None),
        rollout_config=RolloutConfig(max_tokens_to_generate=a.max_new_tokens, max_prompt_length=prompt_len, temperature=0.9, top_p=1.0,
                                     top_k=50, kv_cache_size=prompt_len + a.max_new_tokens + 8, eos_tokens=[tok.eos_id()])))
    learner = GRPOLearner(cluster, [gsm8k_vtc.vtc_reward_fn], GRPOConfig(num_generations=a.generations, beta=0.0, epsilon=0.2),
                          metric_fns=[gsm8k_vtc.vtc_metric_fn])
    learner.train(train)
    lg = cluster.metrics_logger
    out = {"steps": int(cluster.global_steps),
           "reward_mean": [float(x) for x in lg.get_metric_history("", "rewards/score/mean", "train")],
           "solve_ratio": [float(x) for x in lg.get_metric_history("", "rewards/solve_ratio", "train")]}
    print(json.dumps(out))
    if tmp is not None:
        tmp.cleanup()
    return out


if __name__ == "__main__":
    main()
