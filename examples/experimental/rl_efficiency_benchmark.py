"""Wall-clock comparison of the two RL stacks on the same multi-turn task
(the job of tunix/experimental/examples/rl_efficiency_benchmark/{benchmark,runtime}.py).

    PYTHONPATH=. python examples/experimental/rl_efficiency_benchmark.py [--steps 3] [--prompts 4] [--group-size 4] [--workers 2]

Both arms train the same randomly initialised toy decoder with GRPO on FrozenLake episodes (the environment's reward,
the model's tokens only in the loss), for the same number of steps, prompts per step and generations per prompt:

  agentic      `rl.agentic.AgenticGRPOLearner`: one process, episodes as coroutines against the cluster's own sampler,
               groups trained on as they complete, weight sync under the rollout lock;
  distributed  `experimental.orchestrator.StandardRLProgram` over a `DistributedRLEngine`: episode workers
               (`AgenticRolloutWorker`, each with its own sampler over a copy of the model that weight sync refreshes), a
               split-step trainer worker, dispatch / poll / critique / train stages overlapping on one event loop.

It prints one JSON line per arm (seconds per step, episodes per second, reward mean of the last step) and their ratio.
With a random toy model on CPU the numbers compare the stacks' overheads, not learning; on a GPU pass `--device cuda`."""
import argparse
import asyncio
import copy
import json
import time

import torch

from tunix_b200 import optim
from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig, CacheConfig, TrainingConfig
from tunix_b200.experimental.common.datatypes import GenerationArgs, Role
from tunix_b200.experimental.orchestrator.algorithm_adapter import GRPOAdapter, env_reward
from tunix_b200.experimental.orchestrator.batch_assembly import BatchConfig
from tunix_b200.experimental.orchestrator.distributed_rl_engine import DistributedRLEngine
from tunix_b200.experimental.orchestrator.rl_program import StandardRLProgram
from tunix_b200.experimental.rollout.sampler import EngineSamplerAdapter
from tunix_b200.experimental.train.peft_trainer_v2 import TrainerV2
from tunix_b200.experimental.worker.agentic_rollout_worker import AgenticRolloutWorker
from tunix_b200.experimental.worker.factories import ByteTokenizer, toy_config
from tunix_b200.experimental.worker.trainer_worker import TrainerWorker
from tunix_b200.generate.sampler import Sampler
from tunix_b200.models.transformer import create_model
from tunix_b200.rl.agentic.agentic_grpo_learner import AgenticGRPOLearner
from tunix_b200.rl.agentic.environments.frozenlake_environment import FrozenLakeAgent, FrozenLakeEnv
from tunix_b200.rl.agentic.parser.chat_template_parser import get_parser
from tunix_b200.rl.algorithm_config import GRPOConfig
from tunix_b200.rl.rl_cluster import RLCluster
from tunix_b200.sft.peft_trainer import PeftTrainer
from tunix_b200.sft.utils import LossOutput, WeightedMetric

MAX_TURNS, RESPONSE_BUDGET, KV = 3, 48, 1024      # the budget covers the model's and the environment's tokens of an episode


def _config():
    return toy_config().replace(max_position=2048)


def tasks(n: int, steps: int) -> list:
    return [[{"seed": 100 * s + i, "size": 4, "p": 0.8, "max_steps": MAX_TURNS} for i in range(n)] for s in range(steps)]


def pg_loss(model, input_tokens, completion_mask, advantages, segment_ids=None, positions=None, **_):
    hidden, _ = model(input_tokens[:, :-1], positions=None if positions is None else positions[:, :-1],
                      segment_ids=None if segment_ids is None else segment_ids[:, :-1], skip_lm_head=True)
    lp = model.token_logprobs(hidden.reshape(-1, hidden.shape[-1]), input_tokens[:, 1:].reshape(-1).long())[0]
    m = completion_mask[:, 1:]
    return LossOutput(loss=WeightedMetric(-(lp.view(input_tokens.shape[0], -1) * advantages[:, 1:] * m).sum(), m.sum()))


def run_agentic(a, device) -> dict:
    tok = ByteTokenizer()
    actor = create_model(_config(), seed=0).to(device)
    tc = RLTrainingConfig(eval_every_n_steps=10 ** 9, max_steps=a.steps, actor_optimizer=optim.AdamW(1e-4), mini_batch_size=a.prompts,
                          train_micro_batch_size=a.group_size)
    rc = RolloutConfig(max_tokens_to_generate=RESPONSE_BUDGET, max_prompt_length=512, temperature=1.0, seed=1, kv_cache_size=KV,
                       eos_tokens=[tok.eos_id()])
    cl = RLCluster(actor=actor, tokenizer=tok, cluster_config=ClusterConfig(role_to_mesh={}, training_config=tc, rollout_config=rc))
    learner = AgenticGRPOLearner(cl, [], GRPOConfig(num_generations=a.group_size, beta=0.0), agent_class=FrozenLakeAgent,
                                 env_class=FrozenLakeEnv, chat_parser=get_parser("qwen"), max_turns=MAX_TURNS, max_concurrency=64)
    data = [{"tasks": batch} for batch in tasks(a.prompts, a.steps)]
    t0 = time.perf_counter()
    learner.train(data)
    dt = time.perf_counter() - t0
    hist = cl.metrics_logger.get_metric_history("", "rewards/score/mean", "train")
    return {"arm": "agentic", "steps": int(cl.global_steps), "seconds_per_step": dt / max(cl.global_steps, 1),
            "episodes_per_s": a.steps * a.prompts * a.group_size / dt, "reward_mean_last": float(hist[-1]) if len(hist) else None}


def run_distributed(a, device) -> dict:
    tok = ByteTokenizer()
    actor = create_model(_config(), seed=0).to(device)
    trainer = PeftTrainer(actor, optim.AdamW(1e-4), TrainingConfig(eval_every_n_steps=10 ** 9, pbar_description=None,
                                                                   resume_from_checkpoint_on_init=False))
    trainer.with_loss_fn(pg_loss).with_gen_model_input_fn(
        lambda b: {k: (torch.as_tensor(v).long() if k == "input_tokens" else torch.as_tensor(v)).to(device) for k, v in b.items()})
    workers = []
    for i in range(a.workers):
        replica = copy.deepcopy(actor)

        def apply(version, payload, m=replica):
            m.load_state_dict(payload)
        sampler = EngineSamplerAdapter(Sampler(replica, tok, CacheConfig(KV, _config().num_layers, _config().num_kv_heads,
                                                                         _config().head_dim)), tokenizer=tok, eos_tokens=[tok.eos_id()],
                                       batch_window_s=0.002)
        workers.append(AgenticRolloutWorker(f"episodes-{i}", sampler, tok, chat_parser=get_parser("qwen"), eos_ids=[tok.eos_id()],
                                            default_agent=FrozenLakeAgent, default_env=FrozenLakeEnv, apply_weights=apply))
    tw = TrainerWorker("trainer-0", TrainerV2(trainer))
    for w in workers + [tw]:
        w.start()
    eng = DistributedRLEngine(workers, {Role.ACTOR: tw}, export_weights=lambda: {k: v.detach().clone() for k, v in actor.state_dict().items()})
    data = [{"prompt_id": f"lake-{s}-{i}", "task": t, "max_turns": MAX_TURNS, "max_response_length": RESPONSE_BUDGET} for s, batch in enumerate(tasks(a.prompts, a.steps))
            for i, t in enumerate(batch)]
    prog = StandardRLProgram(GRPOAdapter(reward_fn=env_reward, drop_uniform_groups=False), data, a.steps, num_generations=a.group_size,
                             batch_size=a.prompts, batch_config=BatchConfig(rows_per_microbatch=a.group_size, max_packed_len=a.packed_len,
                                                                            max_prompt_length=1024, max_response_length=1024),
                             generation_args=GenerationArgs(max_tokens=RESPONSE_BUDGET, temperature=1.0), checkpoint_every=0,
                             poll_timeout_s=0.05)
    t0 = time.perf_counter()
    hist = prog.run(eng)
    dt = time.perf_counter() - t0
    asyncio.run(eng.close())
    for w in workers + [tw]:
        w.stop()
    return {"arm": "distributed", "steps": len(hist), "seconds_per_step": dt / max(len(hist), 1),
            "episodes_per_s": sum(h["num_rollouts"] for h in hist) / dt, "reward_mean_last": hist[-1]["reward_mean"] if hist else None,
            "padding_ratio": hist[-1].get("padding_ratio") if hist else None}


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--prompts", type=int, default=4)
    ap.add_argument("--group-size", type=int, default=4)
    ap.add_argument("--workers", type=int, default=2)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--packed-len", type=int, default=1024, help="tokens per packed training row of the distributed arm")
    ap.add_argument("--arms", default="agentic,distributed")
    a = ap.parse_args(argv)
    device = torch.device(a.device)
    out = {}
    for arm in a.arms.split(","):
        out[arm] = {"agentic": run_agentic, "distributed": run_distributed}[arm](a, device)
        print(json.dumps(out[arm]))
    if len(out) == 2:
        print(json.dumps({"distributed_over_agentic_seconds_per_step": out["distributed"]["seconds_per_step"] / out["agentic"]["seconds_per_step"]}))
    return out


if __name__ == "__main__":
    main()
