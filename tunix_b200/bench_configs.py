"""Runners for the benchmark configurations other than the headline SFT one (which is `bench.py`):

    python -m tunix_b200.bench_configs tiny_lora_cpu
    python -m tunix_b200.bench_configs grpo  [--layers L] [--prompts P] [--steps S]      (torchrun for > 1 GPU)
    python -m tunix_b200.bench_configs dpo   [--layers L] [--pairs N]
    python -m tunix_b200.bench_configs moe   [--layers L]                                (torchrun; experts over ranks)

All use synthetic uniform token ids and random-init weights. `--layers` shrinks a model so that a configuration
fits fewer GPUs than it was specified for; the JSON line names the layer count that actually ran, so a reduced
run cannot be mistaken for the full one. Times are CUDA-event times, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist


class IdTokenizer:
    """Token ids written as space-separated integers: lets string-based APIs carry synthetic ids."""

    def __init__(self, vocab: int, eos: int = -1, pad: int = 0, bos=None):
        self.vocab, self._eos, self._pad, self._bos = vocab, eos, pad, bos

    def encode(self, s, **_):
        return [int(t) for t in s.split()] if isinstance(s, str) else list(s)

    def decode(self, ids, **_):
        return " ".join(str(int(i)) for i in ids)

    def bos_id(self):
        return self._bos

    def eos_id(self):
        return self._eos

    def pad_id(self):
        return self._pad


def _dist():
    if "RANK" in os.environ and not dist.is_initialized():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl")
    return (dist.get_rank(), dist.get_world_size()) if dist.is_initialized() else (0, 1)


def _max_over_ranks(x: float, dev) -> float:
    if not dist.is_initialized():
        return x
    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def tiny_lora_cpu(args) -> dict:
    """Config 1: tiny Llama-style decoder, fp32, LoRA r=8 on q/v, 20 AdamW steps, against a plain PyTorch oracle."""
    from . import lora, optim
    from .common.configs import TrainingConfig
    from .models.config import ModelConfig
    from .models.transformer import create_model
    from .sft.peft_trainer import PeftTrainer, TrainingInput
    cfg = ModelConfig(family="llama3", num_layers=2, vocab_size=1024, embed_dim=256, hidden_dim=1024, num_heads=4, head_dim=64,
                      num_kv_heads=2, norm_eps=1e-6, rope_theta=10000.0, dtype=torch.float32, max_position=128)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, 1024, (4, 128), generator=g)
    mask = torch.zeros(4, 128)
    mask[:, 64:] = 1

    def run(native: bool):
        model = create_model(cfg, seed=0)
        lora.apply_lora_to_model(model, lora.LoraProvider(module_path=r".*(q_proj|v_proj)", rank=8, alpha=16.0), seed=0)
        if native:
            tr = PeftTrainer(model, optim.AdamW(1e-3, weight_decay=0.0), TrainingConfig(eval_every_n_steps=10 ** 9, max_steps=20,
                                                                                         pbar_description=None))
            tr.train([TrainingInput(toks, mask)] * 20)
            return tr.metrics_logger.get_metric_history("", "loss", "train")
        params = [p for n, p in model.named_parameters() if "lora_" in n]
        for n, p in model.named_parameters():
            p.requires_grad_("lora_" in n)
        opt = torch.optim.AdamW(params, lr=1e-3, weight_decay=0.0, betas=(0.9, 0.999), eps=1e-8)
        losses = []
        for _ in range(20):
            logits = model(toks)[0].float()
            lp = torch.log_softmax(logits[:, :-1], -1).gather(-1, toks[:, 1:, None].long()).squeeze(-1)
            loss = -(lp * mask[:, 1:]).sum() / mask[:, 1:].sum()
            opt.zero_grad()
            loss.backward()
            opt.step()
            losses.append(float(loss))
        return losses
    ours, oracle = run(True), run(False)
    return {"config": "tiny_lora_cpu", "steps": 20, "loss_first": ours[0], "loss_last": ours[-1],
            "max_abs_diff_vs_pytorch_fp32": float(np.max(np.abs(np.asarray(ours) - np.asarray(oracle))))}


def grpo(args) -> dict:
    """Config 3: Qwen3-8B GRPO, 64 prompts x 8 generations, prompt 256, up to 768 sampled tokens, the sampler's weights
    refreshed from the actor's after every update.

    --layout colocated      every rank hosts actor (sharded optimizer), reference (row-sharded, gathered inside the
                            GEMMs, unless --replicated-reference) and a sampler copy of its own
    --layout disaggregated  the first half of the ranks trains, the second half hosts the sampler: generation of the
                            next batch overlaps the update, weights cross NVLink peer to peer (`rl/reshard.py`)"""
    from . import optim
    from .common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
    from .common.datatypes import Role
    from .models.config import get_config
    from .models.transformer import create_model
    from .rl.algorithm_config import GRPOConfig
    from .rl.grpo.grpo_learner import GRPOLearner
    from .rl.placement import RolePlacement
    from .rl.rl_cluster import RLCluster
    rank, world = _dist()
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = get_config("qwen3_8b").replace(dtype=torch.bfloat16, max_position=1032)
    if args.layers:
        cfg = cfg.replace(num_layers=args.layers)
    disagg = args.layout == "disaggregated" and world >= 2
    r2m = {}
    if disagg:
        half = world // 2
        r2m = {Role.ACTOR: list(range(half)), Role.REFERENCE: list(range(half)), Role.ROLLOUT: list(range(half, world))}
    pl = RolePlacement(r2m)
    n_ctl = len(pl.controllers)
    actor = create_model(cfg, device=dev, seed=0) if pl.has(Role.ACTOR) else None
    ref = None
    if pl.has(Role.REFERENCE):
        ref = create_model(cfg, device=dev, seed=0)
        for p in ref.parameters():
            p.requires_grad_(False)
    sampler = None
    if disagg and pl.has(Role.ROLLOUT):
        sampler = create_model(cfg, device=dev, seed=0)
        for p in sampler.parameters():
            p.requires_grad_(False)
    tok = IdTokenizer(cfg.vocab_size)
    G = 8
    per_rank = max(args.prompts // n_ctl, 1)
    # batch sizes count prompts; every prompt stands for its G generations (a micro-batch of `micro` prompts is
    # micro x G sequences)
    micro = max(1, min(args.micro // G, per_rank))      # --micro counts sequences: 4 -> one prompt = 8 sequences of 1024 tokens
    tcfg = RLTrainingConfig(eval_every_n_steps=10 ** 9, max_steps=args.steps, actor_optimizer=optim.AdamW(1e-6, max_grad_norm=1.0),
                            mini_batch_size=per_rank, train_micro_batch_size=micro, rollout_micro_batch_size=per_rank,
                            compute_logps_micro_batch_size=micro * 2 if per_rank % (micro * 2) == 0 else micro,
                            pbar_description=None)
    rc = RolloutConfig(max_tokens_to_generate=768, max_prompt_length=256, temperature=1.0, top_p=1.0, seed=2,
                       kv_cache_size=1032, eos_tokens=[-1],
                       max_running_requests=min(args.max_running, max(args.prompts // max(world - n_ctl, 1) if disagg else per_rank, 1) * G))
    cluster = RLCluster(actor=actor, reference=ref, rollout_model=sampler, tokenizer=tok, placement=pl,
                        separate_rollout_copy=not disagg,
                        cluster_config=ClusterConfig(role_to_mesh=r2m, training_config=tcfg, rollout_config=rc, rollout_engine="paged",
                                                     shard_frozen_models=not args.replicated_reference))
    out = {"config": "grpo_qwen3_8b", "n_gpus": world, "layers": cfg.num_layers, "layout": pl.layout, "generations": G,
           "reference": "replicated" if args.replicated_reference or world == 1 else "row-sharded (gathered in the GEMMs)"}
    if not cluster.is_controller:
        cluster.serve()
        res = {"sync_s": cluster.last_weight_sync_seconds, "sync_bytes": cluster.last_weight_sync_bytes}
        allres = [None] * world
        dist.all_gather_object(allres, res)
        return out

    def reward(prompts, completions, completion_ids=None, completion_lengths=None, **_):
        res = []
        for ids, n in zip(completion_ids, completion_lengths):
            ids = np.asarray(ids[:int(n)])
            res.append(float((ids % 7 == 0).mean() if len(ids) else 0.0) - 0.001 * float(n))
        return res
    learner = GRPOLearner(cluster, [reward], GRPOConfig(num_generations=G, beta=0.04, epsilon=0.2))
    rng = np.random.default_rng(2 + rank)
    data = [{"prompts": [" ".join(map(str, rng.integers(3, cfg.vocab_size, 256))) for _ in range(per_rank)]}
            for _ in range(args.steps)]
    orig = learner._generate_and_compute_advantage
    roll_t, starts, sync_t = [], [], []

    def timed(*a, **kw):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        starts.append(t0)
        r = orig(*a, **kw)
        torch.cuda.synchronize()
        roll_t.append(time.perf_counter() - t0)
        return r
    learner._generate_and_compute_advantage = timed
    orig_sync = cluster.sync_weights

    def timed_sync():
        orig_sync()
        sync_t.append((cluster.last_weight_sync_seconds, cluster.last_weight_sync_bytes))
    cluster.sync_weights = timed_sync
    torch.cuda.synchronize()
    t_begin = time.perf_counter()
    learner.train(data)                      # a step = rollout + scoring + reference log-probs + update + weight sync
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    bounds = starts + [t_end]
    times = [bounds[i + 1] - bounds[i] for i in range(len(starts))] or [t_end - t_begin]
    mine = {"sync_s": sync_t[-1][0] if sync_t else None, "sync_bytes": sync_t[-1][1] if sync_t else 0,
            "step": times[-1], "first": times[0], "roll": roll_t[-1] if roll_t else None}
    allres = [mine]
    if world > 1:
        allres = [None] * world
        dist.all_gather_object(allres, mine)
    ctl = [r for r in allres if r and "step" in r]
    syncs = [r for r in allres if r and r.get("sync_s")]
    sync_s = max((r["sync_s"] for r in syncs), default=None)
    pulled = max((r["sync_bytes"] for r in syncs), default=0)
    out.update({"prompts": per_rank * n_ctl, "step_seconds": max(r["step"] for r in ctl),
                "first_step_seconds": max(r["first"] for r in ctl),
                "rollout_and_scoring_seconds": max((r["roll"] for r in ctl if r["roll"] is not None), default=None),
                "rollout_tokens_per_step": per_rank * G * 768 * n_ctl,
                "weight_sync_seconds": sync_s, "weight_sync_bytes_per_rank": pulled,
                "weight_sync_gb_per_s_per_rank": (pulled / sync_s / 1e9) if sync_s and pulled else None,
                "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30})
    return out


def dpo(args) -> dict:
    """Config 4: Gemma-2-9B DPO with LoRA r=16 on all linear layers, 32 pairs of 512 + 512 tokens per step."""
    from . import lora, optim
    from .models.config import get_config
    from .models.transformer import create_model
    from .sft.dpo.dpo_trainer import DPOTrainer, DPOTrainingConfig, TrainingInput
    rank, world = _dist()
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = get_config("gemma2_9b").replace(dtype=torch.bfloat16, max_position=1024)
    if args.layers:
        cfg = cfg.replace(num_layers=args.layers)
    model = create_model(cfg, device=dev, seed=0)
    lora.apply_lora_to_model(model, lora.LoraProvider(rank=16, alpha=32.0), seed=0)
    pairs = max(args.pairs // world, 1)
    tc = DPOTrainingConfig(eval_every_n_steps=10 ** 9, max_steps=args.steps, beta=0.1, max_prompt_length=512, max_response_length=512,
                           pbar_description=None, gradient_accumulation_steps=max(pairs // args.micro, 1))
    opt = optim.AdamW(5e-6)
    if world > 1:          # data parallel: adapter gradients summed and the Adam state split over the ranks
        from .parallel import fsdp
        opt = fsdp.shard_optimizer(opt)
    tr = DPOTrainer(model, None, opt, tc)
    g = torch.Generator().manual_seed(3 + rank)
    mb = min(args.micro, pairs)

    def batch():
        def ids(n):
            return torch.randint(3, cfg.vocab_size, (mb, n), generator=g)
        ones = torch.ones(mb, 512)
        return TrainingInput(prompt_ids=ids(512), prompt_mask=ones, chosen_ids=ids(512), chosen_mask=ones, rejected_ids=ids(512),
                             rejected_mask=ones)
    accum = max(pairs // mb, 1)
    times = []
    for step in range(args.steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(accum):
            tr._train_step(tr._prepare_inputs(batch()), i == accum - 1)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / 1e3)
    return {"config": "dpo_gemma2_9b_lora", "n_gpus": world, "layers": cfg.num_layers, "pairs_per_step": pairs * world,
            "step_seconds": _max_over_ranks(float(np.median(times[1:] or times)), dev),
            "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30}


def moe(args) -> dict:
    """Config 5: Qwen3-30B-A3B SFT with the experts spread over the ranks, global batch 32 x 4096."""
    from . import optim
    from .common.configs import TrainingConfig
    from .models.config import get_config
    from .models.transformer import create_model
    from .parallel import ep as ep_lib
    from .sft.peft_trainer import PeftTrainer, TrainingInput
    rank, world = _dist()
    dev = torch.device("cuda", torch.cuda.current_device())
    from .models.config import RematConfig
    # per-layer recompute: the permuted expert activations of 48 layers do not fit next to the optimizer state
    cfg = get_config("qwen3_30b_a3b").replace(dtype=torch.bfloat16, max_position=4096, router_aux_loss_coef=0.001,
                                              remat_config=RematConfig.DECODER)
    if args.layers:
        cfg = cfg.replace(num_layers=args.layers)
    model = create_model(cfg, device=dev, seed=0)
    if world > 1:
        ep_lib.shard_experts(model, ep_lib.EPContext(device=dev, capacity_factor=args.ep_capacity or None))
    seqs = max(32 // world, 1)
    mb = min(args.micro, seqs)
    tr = PeftTrainer(model, optim.AdamW(2e-5, max_grad_norm=1.0),
                     TrainingConfig(eval_every_n_steps=10 ** 9, max_steps=args.steps, pbar_description=None,
                                    gradient_accumulation_steps=seqs // mb))
    g = torch.Generator().manual_seed(4 + rank)
    times = []
    for step in range(args.steps):
        batches = [{"input_tokens": torch.randint(0, cfg.vocab_size, (mb, 4096), generator=g).to(dev, torch.int32),
                    "input_mask": torch.ones(mb, 4096, device=dev), "_is_local_shard": True} for _ in range(seqs // mb)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i, b in enumerate(batches):
            tr._train_step(b, i == len(batches) - 1)
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            model.dp_shard.raise_if_overflow()
        times.append(e0.elapsed_time(e1) / 1e3)
    sec = _max_over_ranks(float(np.median(times[1:] or times)), dev)
    return {"config": "moe_qwen3_30b_a3b_sft", "n_gpus": world, "layers": cfg.num_layers, "global_batch": seqs * world, "seq_len": 4096,
            "ep_capacity_factor": (args.ep_capacity or None) if world > 1 else None,
            "step_seconds": sec, "tokens_per_sec": seqs * world * 4096 / sec, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", choices=["tiny_lora_cpu", "grpo", "dpo", "moe"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--prompts", type=int, default=64)
    ap.add_argument("--pairs", type=int, default=32)
    ap.add_argument("--micro", type=int, default=4)
    ap.add_argument("--ep-capacity", type=float, default=0.0,
                    help="moe: receive buffers of the expert-parallel exchange sized as this multiple of the even share, "
                         "which needs no host read-back per layer (overflow is flagged and raises at the end of the step); "
                         "0 = exact sizes read back from the device every layer")
    ap.add_argument("--max-running", type=int, default=256, help="sequences decoded together by the rollout engine")
    ap.add_argument("--layout", default="colocated", choices=["colocated", "disaggregated"], help="grpo: where the sampler lives")
    ap.add_argument("--replicated-reference", action="store_true", help="grpo: keep the reference model whole on every rank")
    args = ap.parse_args(argv)
    limit = os.environ.get("TUNIX_B200_DUMP_STACKS_AFTER")
    if limit:
        # a run that is still going after this many seconds prints the Python stack of every thread of every rank
        # and exits: where a multi-rank configuration waits, without holding the GPUs until an outer timeout
        import faulthandler
        faulthandler.dump_traceback_later(float(limit), exit=True)
    res = {"tiny_lora_cpu": tiny_lora_cpu, "grpo": grpo, "dpo": dpo, "moe": moe}[args.config](args)
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(json.dumps(res))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
