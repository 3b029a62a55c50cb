"""Worker of the 2-GPU placement test (run under torch.distributed.run): rank 0 trains the actor, rank 1 hosts the
sampler on the paged engine; the weights reach it through the peer-to-peer reshard kernel."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    out_path = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from tunix_b200 import _lib, optim
    from tunix_b200.bench_configs import IdTokenizer
    from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
    from tunix_b200.common.datatypes import Role
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.rl.algorithm_config import GRPOConfig
    from tunix_b200.rl.grpo.grpo_learner import GRPOLearner
    from tunix_b200.rl.placement import RolePlacement
    from tunix_b200.rl.rl_cluster import RLCluster
    cfg = ModelConfig(family="qwen3", num_layers=2, vocab_size=2048, embed_dim=512, hidden_dim=1024, num_heads=4, head_dim=128,
                      num_kv_heads=2, qk_norm=True, dtype=torch.bfloat16, max_position=256)
    r2m = {Role.ACTOR: [0], Role.REFERENCE: [0], Role.ROLLOUT: [1]}
    pl = RolePlacement(r2m)
    actor = create_model(cfg, device=dev, seed=0) if rank == 0 else None
    ref = create_model(cfg, device=dev, seed=0) if rank == 0 else None
    sampler = create_model(cfg, device=dev, seed=7) if rank == 1 else None      # other weights: the sync must replace them
    tc = RLTrainingConfig(eval_every_n_steps=10 ** 9, max_steps=2, actor_optimizer=optim.AdamW(1e-3, weight_decay=0.0),
                          mini_batch_size=8, train_micro_batch_size=4, pbar_description=None)
    rc = RolloutConfig(max_tokens_to_generate=24, max_prompt_length=16, temperature=1.0, top_p=1.0, seed=2, kv_cache_size=64,
                       eos_tokens=[-1], max_running_requests=16)
    cl = RLCluster(actor=actor, reference=ref, rollout_model=sampler, tokenizer=IdTokenizer(cfg.vocab_size), placement=pl,
                   cluster_config=ClusterConfig(role_to_mesh=r2m, training_config=tc, rollout_config=rc, rollout_engine="paged"))
    res = {"controller": cl.is_controller}
    if not cl.is_controller:
        res["served"] = cl.serve()
        w = torch.cat([p.detach().float().reshape(-1) for p in cl.rollout_actor.parameters()])
    else:
        def reward(prompts, completions, completion_ids=None, completion_lengths=None, **_):
            return [float((np.asarray(i[:int(n)]) % 7 == 0).mean()) for i, n in zip(completion_ids, completion_lengths)]
        learner = GRPOLearner(cl, [reward], GRPOConfig(num_generations=2, beta=0.04))
        rng = np.random.default_rng(3)
        data = [{"prompts": [" ".join(map(str, rng.integers(3, cfg.vocab_size, 16))) for _ in range(4)]} for _ in range(2)]
        learner.train(data)
        res.update(steps=cl.global_steps, rounds=cl.exchange.rounds)
        w = torch.cat([p.detach().float().reshape(-1) for p in actor.parameters()])
    torch.cuda.synchronize()
    _lib.raise_if_kernel_error()
    res["sync_s"], res["sync_bytes"] = cl.last_weight_sync_seconds, cl.last_weight_sync_bytes
    res["fused"] = bool(getattr(cl._resharder, "fused", False))
    ws = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(ws, w)
    res["max_abs_diff"] = float((ws[0] - ws[1]).abs().max())
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        json.dump(allres, open(out_path, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
