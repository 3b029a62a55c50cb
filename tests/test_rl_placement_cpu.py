"""Role placement in the RL stack on CPU ranks (gloo): the layouts `ClusterConfig.role_to_mesh` can describe.

* colocated with a sampler copy of its own: every rank trains on its own prompts through the sharded optimizer,
  and the sampler's copy equals the actor's weights after every weight sync;
* disaggregated: ranks 0-1 hold the actor and run the loop, rank 2 holds the sampler, rank 3 the reference; the
  last two sit in `serve()`; generation of batch k+1 is requested before the update on batch k.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg():
    from tunix_b200.models.config import ModelConfig
    return ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2,
                                            head_dim=16, num_kv_heads=1)


def _reward(prompts, completions, completion_ids=None, completion_lengths=None, **kw):
    return [float((np.asarray(ids[:n]) % 7 == 0).mean()) if n else 0.0 for ids, n in zip(completion_ids, completion_lengths)]


def _run(rank, world, port, layout, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tests.test_sampler_cpu import CharTok
    from tunix_b200 import optim
    from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
    from tunix_b200.common.datatypes import Role
    from tunix_b200.models.transformer import create_model
    from tunix_b200.rl.algorithm_config import GRPOConfig
    from tunix_b200.rl.grpo.grpo_learner import GRPOLearner
    from tunix_b200.rl.placement import RolePlacement
    from tunix_b200.rl.rl_cluster import RLCluster
    if layout == "colocated":
        r2m = {}
    elif layout == "halves":        # trainer half (actor + reference together), sampler half
        r2m = {Role.ACTOR: [0, 1], Role.REFERENCE: [0, 1], Role.ROLLOUT: [2, 3]}
    else:
        r2m = {Role.ACTOR: [0, 1], Role.ROLLOUT: [2], Role.REFERENCE: [3]}
    pl = RolePlacement(r2m)
    tc = RLTrainingConfig(eval_every_n_steps=1000, max_steps=3, actor_optimizer=optim.AdamW(1e-2, weight_decay=0.0),
                          mini_batch_size=2, train_micro_batch_size=1)
    rc = RolloutConfig(max_tokens_to_generate=6, max_prompt_length=8, temperature=1.0, top_p=1.0, seed=3, kv_cache_size=32,
                       eos_tokens=[63])
    cc = ClusterConfig(role_to_mesh=r2m, training_config=tc, rollout_config=rc)
    mk = lambda seed: create_model(_cfg(), seed=seed)  # noqa: E731
    actor = mk(0) if pl.has(Role.ACTOR) else None
    # the sampler starts from DIFFERENT weights: only a working sync makes it follow the actor
    sampler = mk(5) if (pl.has(Role.ROLLOUT) and layout != "colocated") else None
    ref = mk(0) if pl.has(Role.REFERENCE) else None
    cl = RLCluster(actor=actor, reference=ref, rollout_model=sampler, tokenizer=CharTok(), cluster_config=cc, placement=pl,
                   separate_rollout_copy=(layout == "colocated"))
    res = {"layout": pl.layout, "controller": cl.is_controller}
    if not cl.is_controller:
        res["served"] = cl.serve()
        if cl.rollout_actor is not None:
            res["sampler"] = torch.cat([p.detach().reshape(-1) for p in cl.rollout_actor.parameters()])
    else:
        learner = GRPOLearner(cl, [_reward], GRPOConfig(num_generations=2, beta=0.04))
        data = [{"prompts": [f"{chr(97 + rank)}{chr(98 + s)}", f"{chr(99 + rank)}{chr(100 + s)}"]} for s in range(3)]
        learner.train(data)
        res["steps"] = cl.global_steps
        res["sharded"] = bool(getattr(cl.actor_trainer.optimizer, "is_sharded", False))
        res["actor"] = torch.cat([p.detach().reshape(-1) for p in actor.parameters()])
        if cl.rollout_actor is not None:
            res["sampler"] = torch.cat([p.detach().reshape(-1) for p in cl.rollout_actor.parameters()])
        res["sync_s"] = cl.last_weight_sync_seconds
        res["rounds"] = cl.exchange.rounds
        res["rewards"] = cl.metrics_logger.get_metric_history("", "rewards/score/mean", "train").tolist()
    torch.save(res, f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_colocated_layout_with_a_sampler_copy_of_its_own(tmp_path):
    out = str(tmp_path / "r")
    mp.spawn(_run, args=(2, 29751, "colocated", out), nprocs=2, join=True)
    res = [torch.load(f"{out}.{r}") for r in range(2)]
    assert all(r["layout"] == "colocated" and r["controller"] and r["steps"] == 3 and r["sharded"] for r in res)
    # data parallel: both ranks hold the same actor, and each sampler copy follows it
    assert torch.equal(res[0]["actor"], res[1]["actor"])
    for r in res:
        assert torch.equal(r["sampler"], r["actor"]) and r["sync_s"] is not None
    fresh = torch.cat([p.detach().reshape(-1) for p in __import__("tunix_b200.models.transformer", fromlist=["x"]).create_model(_cfg(), seed=0).parameters()])
    assert not torch.equal(fresh, res[0]["actor"])            # training moved the weights


def test_disaggregated_layout_with_serving_ranks(tmp_path):
    out = str(tmp_path / "r")
    mp.spawn(_run, args=(4, 29753, "disaggregated", out), nprocs=4, join=True)
    res = [torch.load(f"{out}.{r}") for r in range(4)]
    assert [r["layout"] for r in res] == ["disaggregated"] * 4
    assert [r["controller"] for r in res] == [True, True, False, False]
    assert res[0]["steps"] == res[1]["steps"] == 3 and res[0]["sharded"]
    assert torch.equal(res[0]["actor"], res[1]["actor"])
    # the sampler on rank 2 started from other weights and ends with the actor's: the sync crossed ranks
    assert torch.allclose(res[2]["sampler"], res[0]["actor"], atol=1e-6)
    # per step: one generation round and one reference round; the serving ranks saw all of them
    assert res[2]["served"] == res[3]["served"] == 6 and res[0]["rounds"] == 6
    assert len(res[0]["rewards"]) == 3


def _run_groups(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from tunix_b200.common.datatypes import Role
    from tunix_b200.parallel.mesh import Mesh
    from tunix_b200.rl.placement import RoleExchange, RolePlacement
    # rank 0 trains; ranks 1-4 sample as two tensor-parallel groups of two
    pl = RolePlacement({Role.ACTOR: [0], Role.ROLLOUT: Mesh((2, 2), ("fsdp", "tp"), ranks=[1, 2, 3, 4])})
    assert pl.replica_groups(Role.ROLLOUT) == [[1, 2], [3, 4]] and pl.replica_groups(Role.ACTOR) == [[0]]
    ex = RoleExchange(pl)
    seen = []

    def handler(items):
        seen.append(list(items))
        return [(it, rank) for it in items]

    ex.register(Role.ROLLOUT, "generate", handler)
    if pl.is_controller:
        got = ex.call(Role.ROLLOUT, "generate", [10, 11, 12, 13, 14])
        ex.stop()
        torch.save({"got": got}, f"{out}.{rank}")
    else:
        ex.serve()
        torch.save({"seen": seen}, f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_exchange_hands_a_tensor_parallel_group_the_same_items(tmp_path):
    out = str(tmp_path / "g")
    mp.spawn(_run_groups, args=(5, 29787, out), nprocs=5, join=True)
    got = torch.load(out + ".0")["got"]
    # five items over two groups: 3 + 2; the leader of each group (ranks 1 and 3) reports
    assert got == [(10, 1), (11, 1), (12, 1), (13, 3), (14, 3)]
    seen = [torch.load(out + f".{r}")["seen"] for r in range(1, 5)]
    assert seen[0] == seen[1] == [[10, 11, 12]] and seen[2] == seen[3] == [[13, 14]]


def test_halves_layout_trainers_and_samplers(tmp_path):
    """The first half of the ranks hosts actor and reference, the second half two samplers."""
    out = str(tmp_path / "r")
    mp.spawn(_run, args=(4, 29757, "halves", out), nprocs=4, join=True)
    res = [torch.load(f"{out}.{r}") for r in range(4)]
    assert [r["controller"] for r in res] == [True, True, False, False]
    assert res[0]["steps"] == res[1]["steps"] == 3 and torch.equal(res[0]["actor"], res[1]["actor"])
    for r in (2, 3):
        assert torch.allclose(res[r]["sampler"], res[0]["actor"], atol=1e-6)
