"""GSM8K GRPO on the distributed stack (the job of tunix/experimental/examples/math_gsm8k_dist/run_gsm8k_dist_grpo.py).

    PYTHONPATH=. python examples/experimental/gsm8k_distributed.py --tiny --steps 2          # toy model, sample data, CPU
    PYTHONPATH=. python examples/experimental/gsm8k_distributed.py --data /data/gsm8k --model qwen3-1.7b --model-path /ckpt/Qwen3-1.7B

Rollout workers (one sampler each over a copy of the model; on a GPU put them on their own devices with `--rollout-devices`)
answer single-call requests, the program scores groups with the VTC reward (`utils/gsm8k_vtc.py`), packs the
trajectories and drives a split-step trainer worker; weights go to the rollout workers after every step and the
consumed trajectories are written to an ATIF store (`--store DIR`)."""
import argparse
import asyncio
import copy
import json
import os
import tempfile

import torch

from tunix_b200 import optim
from tunix_b200.common.configs import CacheConfig, TrainingConfig
from tunix_b200.experimental.common.datatypes import GenerationArgs, Role
from tunix_b200.experimental.orchestrator.algorithm_adapter import GRPOAdapter
from tunix_b200.experimental.orchestrator.batch_assembly import BatchConfig
from tunix_b200.experimental.orchestrator.distributed_rl_engine import DistributedRLEngine
from tunix_b200.experimental.orchestrator.rl_program import StandardRLProgram
from tunix_b200.experimental.train.peft_trainer_v2 import TrainerV2
from tunix_b200.experimental.trajectory.file_store import FileTrajectoryStore
from tunix_b200.experimental.worker.rollout_worker import RolloutWorker
from tunix_b200.experimental.worker.trainer_worker import TrainerWorker
from tunix_b200.generate.sampler import Sampler
from tunix_b200.sft.peft_trainer import PeftTrainer
from tunix_b200.sft.utils import LossOutput, WeightedMetric
from tunix_b200.utils import gsm8k_vtc, script_utils

from examples.rl.grpo_gsm8k_vtc import _SAMPLE, build_model


def pg_loss(model, input_tokens, completion_mask, advantages, segment_ids=None, positions=None, **_):
    hidden, _ = model(input_tokens[:, :-1], positions=None if positions is None else positions[:, :-1],
                      segment_ids=None if segment_ids is None else segment_ids[:, :-1], skip_lm_head=True)
    lp = model.token_logprobs(hidden.reshape(-1, hidden.shape[-1]), input_tokens[:, 1:].reshape(-1).long())[0]
    m = completion_mask[:, 1:]
    return LossOutput(loss=WeightedMetric(-(lp.view(input_tokens.shape[0], -1) * advantages[:, 1:] * m).sum(), m.sum()))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--data", default=None)
    ap.add_argument("--model", default="qwen3-1.7b")
    ap.add_argument("--model-path", default=None)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--prompts", type=int, default=8, help="prompt groups per optimizer step")
    ap.add_argument("--generations", type=int, default=8)
    ap.add_argument("--max-new-tokens", type=int, default=512)
    ap.add_argument("--workers", type=int, default=2)
    ap.add_argument("--rollout-devices", default=None, help="comma-separated devices of the rollout workers, e.g. cuda:1,cuda:2")
    ap.add_argument("--max-staleness", type=int, default=0)
    ap.add_argument("--store", default=None, help="directory of the ATIF trajectory store")
    ap.add_argument("--checkpoint-dir", default=None)
    a = ap.parse_args(argv)
    device = torch.device("cuda:0" if torch.cuda.is_available() else "cpu")
    if a.tiny:
        a.prompts, a.generations, a.max_new_tokens = min(a.prompts, 2), min(a.generations, 4), min(a.max_new_tokens, 12)
    tmp = tempfile.TemporaryDirectory()
    if a.data is None:
        a.data = os.path.join(tmp.name, "train.jsonl")
        with open(a.data, "w") as f:
            for q, ans in _SAMPLE * 8:
                f.write(json.dumps({"question": q, "answer": ans}) + "\n")
    records = script_utils.get_dataset(a.data, "train", seed=0, system_prompt="", answer_extractor=gsm8k_vtc.extract_hash_answer)
    actor, tok = build_model(a, device)
    dataset = [{"prompt_id": f"gsm8k-{i}", "prompt_ids": tok.encode(gsm8k_vtc.build_prompt(r["question"])), "answer": r["answer"]}
               for i, r in enumerate(records)]
    longest = max(len(d["prompt_ids"]) for d in dataset)
    cfg = actor.config
    devices = a.rollout_devices.split(",") if a.rollout_devices else [str(device)] * a.workers
    workers = []
    for i, d in enumerate(devices):
        replica = copy.deepcopy(actor).to(d)

        def apply(version, payload, m=replica):
            m.load_state_dict(payload)
        sampler = Sampler(replica, tok, CacheConfig(2 * longest + a.max_new_tokens + 8, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim))
        workers.append(RolloutWorker(f"rollout-{i}", sampler, apply_weights=apply, eos_tokens=[tok.eos_id()]))
    trainer = PeftTrainer(actor, optim.AdamW(1e-6 if not a.tiny else 1e-4, max_grad_norm=1.0),
                          TrainingConfig(eval_every_n_steps=10 ** 9, pbar_description=None, checkpoint_root_directory=a.checkpoint_dir))
    trainer.with_loss_fn(pg_loss).with_gen_model_input_fn(
        lambda b: {k: (torch.as_tensor(v).long() if k == "input_tokens" else torch.as_tensor(v)).to(device) for k, v in b.items()})
    tw = TrainerWorker("trainer-0", TrainerV2(trainer))
    for w in workers + [tw]:
        w.start()
    engine = DistributedRLEngine(workers, {Role.ACTOR: tw}, export_weights=lambda: {k: v.detach().clone() for k, v in actor.state_dict().items()})

    def reward(item, response) -> float:
        return gsm8k_vtc.vtc_completion_outcome(response.text if response.text is not None else tok.decode(response.tokens), item["answer"])[0]
    store = FileTrajectoryStore(a.store) if a.store else None
    program = StandardRLProgram(GRPOAdapter(reward_fn=reward, drop_uniform_groups=not a.tiny), dataset, a.steps, num_generations=a.generations,
                                batch_size=a.prompts, max_staleness=a.max_staleness, trajectory_store=store, poll_timeout_s=0.05,
                                checkpoint_every=1 if a.checkpoint_dir else 0,
                                batch_config=BatchConfig(rows_per_microbatch=4, max_packed_len=max(1024, 2 * (longest + a.max_new_tokens))),
                                generation_args=GenerationArgs(max_tokens=a.max_new_tokens, temperature=0.9, top_k=50))
    history = program.run(engine)
    asyncio.run(engine.close())
    for w in workers + [tw]:
        w.stop()
    if store is not None:
        store.close()
    out = {"steps": len(history), "reward_mean": [h["reward_mean"] for h in history], "loss": [h["loss"] for h in history],
           "padding_ratio": [round(h["padding_ratio"], 3) for h in history], "policy_version": program.policy_version}
    print(json.dumps(out))
    tmp.cleanup()
    return out


if __name__ == "__main__":
    main()
