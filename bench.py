#!/usr/bin/env python
"""Headline benchmark: full-weight SFT tokens/s of Llama-3.1-8B (bf16, fp32 master weights + AdamW state,
grad-clip 1.0, seq 2048, loss on positions >= 512), 8 sequences per GPU (global batch 64 on 8 GPUs).

    python bench.py --gpus N --steps K --warmup W           (N > 1: launched under torch.distributed.run)
    python bench.py --impl reference ...                    (the reference arm; prints why it is unavailable)

Besides the main arm the same process measures, after it, the in-repo baseline of the same step (N > 1: the
sharded optimizer over NCCL collectives; N = 1: stock PyTorch ops in place of this package's kernels), which gives
`vs_baseline`, and a like-for-like scaling point with micro-batch 2 x 4 accumulation steps at every N
(`same_microbatch_value`). `--parallelism zero3` runs the weight-sharded path whose GEMMs gather their weights.

Timing: W (>=3) untimed optimizer steps, then exactly K steps between CUDA events bracketed by a barrier +
synchronize on both sides, max over ranks. Every step streams > 100 GB of weights / optimizer state, far
more than the 126 MB L2, so no explicit flush is needed between iterations. The end-to-end number drives
`PeftTrainer.train` (the public API) with inputs coming from pinned host memory every step and the loss
read back to the host every step. SM clocks and throttle reasons are sampled during the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sft_tokens_per_sec"
SEQ_LEN = 2048
SEQS_PER_GPU = 8
PROMPT_LEN = 512


def reference_arm(args) -> int:
    """The unmodified reference is a JAX/Flax library; none of its dependencies exist offline here."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    why = None
    try:
        import tunix  # noqa: F401
        import jax  # noqa: F401
    except Exception as e:  # ModuleNotFoundError in practice
        why = (f"reference not installable offline: pip --no-index cannot resolve its dependencies "
               f"(jax, flax, optax, orbax, qwix, datasets absent from the offline wheel directory) and --no-deps fails "
               f"in CMake (nanobind missing); import error: {type(e).__name__}: {e}")
    if why is None:
        why = "reference imported but its SFT path needs a JAX GPU backend that is not present"
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}))
    return 0


class ClockSampler:
    """Samples SM clock / throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.samples, self._stop, self._t = gpu_index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.gpu)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._t:
            self._t.join(6)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
                for n, v in zip(names, s[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="llama3p1_8b")
    ap.add_argument("--micro-batch", type=int, default=0, help="sequences per micro-batch (0 = pick from memory)")
    ap.add_argument("--seqs-per-gpu", type=int, default=SEQS_PER_GPU)
    ap.add_argument("--seq-len", type=int, default=SEQ_LEN)
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (debugging only; the "
                    "printed line then names the reduced model and is not the headline)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--parallelism", default="zero2", choices=["zero2", "zero3"],
                    help="N > 1: zero2 = whole bf16 weights, sharded fp32 master / moments, fused reduce-scatter + "
                         "AdamW and overlapped all-gather; zero3 = weights sharded too, every GEMM gathers its weight "
                         "(and reduce-scatters its weight gradient) inside the kernel")
    ap.add_argument("--comm", default="p2p", choices=["p2p", "nccl"],
                    help="zero2 collectives: our peer-memory kernels, or NCCL (the in-repo baseline)")
    ap.add_argument("--arms", default="main,baseline,same_mb",
                    help="comma list. baseline = the same step on the in-repo baseline (N > 1: NCCL collectives; "
                         "N = 1: stock PyTorch ops instead of this package's kernels) -> vs_baseline; same_mb = "
                         "micro-batch 2 x 4 accumulation steps at every N, the like-for-like scaling point")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import contextlib
    import gc

    import torch
    import torch.distributed as dist

    from tunix_b200 import _lib, optim
    from tunix_b200.common.configs import TrainingConfig
    from tunix_b200.models.config import get_config
    from tunix_b200.models.transformer import create_model
    from tunix_b200.ops import functional as F
    from tunix_b200.ops import kernels
    from tunix_b200.sft.peft_trainer import PeftTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    arms = [a for a in args.arms.split(",") if a]

    cfg = get_config(args.model).replace(dtype=torch.bfloat16, max_position=args.seq_len)
    if args.layers:
        cfg = cfg.replace(num_layers=args.layers)
    seqs = args.seqs_per_gpu
    if args.micro_batch > 0:
        main_mb = args.micro_batch
    else:
        # optimizer state + fp32 grads of an unsharded 8B model leave room for ~2 sequences of activations
        main_mb = {1: 2, 2: 4}.get(world, seqs)
    main_mb = min(main_mb, seqs)
    gen = torch.Generator().manual_seed(1234 + rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def run_arm(kind: str, mb: int, steps: int, e2e: bool, sample_clocks: bool):
        """Build model + optimizer + trainer of one arm, warm up, time `steps` optimizer steps; optionally the
        end-to-end pass through `PeftTrainer.train`. Everything of the arm is released before returning."""
        accum = seqs // mb
        torch.manual_seed(0)
        model = create_model(cfg, device=dev, seed=0)
        adam = dict(b1=0.9, b2=0.95, eps=1e-8, weight_decay=0.0, max_grad_norm=1.0)
        ctx = contextlib.nullcontext()
        if kind == "library":
            ctx = F.library_ops()
        if world > 1 and kind == "zero3":
            from tunix_b200.parallel import fsdp3
            fsdp3.apply_weight_sharding(model, fsdp3.CommContext(device=dev))
            opt = optim.AdamW(2e-5, **adam)
        elif world > 1:
            from tunix_b200.parallel import fsdp
            opt = fsdp.ShardedAdamW(2e-5, comm="nccl" if kind == "zero2-nccl" else args.comm, **adam)
        else:
            opt = optim.AdamW(2e-5, **adam)
        tc = TrainingConfig(eval_every_n_steps=10 ** 9, max_steps=None, gradient_accumulation_steps=accum,
                            pbar_description=None, resume_from_checkpoint_on_init=False, max_inflight_computations=2)
        trainer = PeftTrainer(model, opt, tc)
        trainer.is_managed_externally = True

        def host_batch():
            toks = torch.randint(0, cfg.vocab_size, (mb, args.seq_len), generator=gen, dtype=torch.int32).pin_memory()
            mask = torch.zeros(mb, args.seq_len, dtype=torch.float32)
            mask[:, PROMPT_LEN:] = 1
            return {"input_tokens": toks, "input_mask": mask.pin_memory(), "_is_local_shard": True}

        trainer.gen_model_input_fn = lambda b: {k: v for k, v in b.items() if not k.startswith("_")}
        dev_batches = [{k: (v.to(dev, non_blocking=True) if hasattr(v, "to") else v) for k, v in host_batch().items()}
                       for _ in range(accum)]

        def one_step():
            for i in range(accum):
                trainer._train_step(dev_batches[i], is_update_step=(i == accum - 1))

        out = {"micro_batch": mb, "grad_accum": accum}
        with ctx:
            for _ in range(warmup):
                one_step()
            barrier()
            sampler = ClockSampler(local_rank)
            if rank == 0 and sample_clocks:
                sampler.start()
            l0 = kernels.launch_count + getattr(opt, "comm_launches", 0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            for _ in range(steps):
                one_step()
            trainer._params_ready()     # the last step's parameter pulls on the side stream end before e1
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1)
            out["launches"] = int(kernels.launch_count + getattr(opt, "comm_launches", 0) - l0)
            out["clocks"] = sampler.stop() if (rank == 0 and sample_clocks) else None
            out["ms_per_step"] = max_over_ranks(ms) / steps
            if e2e:
                host_batches = [host_batch() for _ in range(steps * accum)]
                h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values() if hasattr(v, "numel")) * accum
                trainer._prev_buffered_train_metrics = None
                trainer._buffered_train_metrics = None
                barrier()
                s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0 = time.perf_counter()
                s0.record()
                trainer.train(host_batches)          # H2D of every batch + delayed loss read-back inside
                s1.record()
                barrier()
                wall_ms = (time.perf_counter() - t0) * 1e3
                e2e_ms = max_over_ranks(max(s0.elapsed_time(s1), wall_ms)) / steps
                # one fp32 loss-sum + one fp32 denominator per micro-batch + the grad-norm per step reach the host
                out["e2e"] = {"ms_per_step": e2e_ms, "h2d_bytes_per_step": int(h2d),
                              "d2h_bytes_per_step": int(8 * accum + 4)}
        _lib.raise_if_kernel_error()
        out["peak_mem_gib"] = torch.cuda.max_memory_allocated() / 2 ** 30
        del trainer, opt, model, dev_batches
        gc.collect()
        torch.cuda.empty_cache()
        return out

    tokens_per_step = seqs * args.seq_len * world
    tps = lambda ms: tokens_per_step / (ms / 1e3)  # noqa: E731
    main_kind = (args.parallelism if args.comm == "p2p" or args.parallelism == "zero3" else "zero2-nccl") if world > 1 \
        else "single"
    main = run_arm(main_kind, main_mb, args.steps, not args.no_e2e, True)
    value = tps(main["ms_per_step"])
    side_steps = max(3, args.steps // 2)

    baseline = None
    if "baseline" in arms and main_kind != "zero2-nccl":
        kind = "zero2-nccl" if world > 1 else "library"
        # the stock-op arm on one GPU keeps more activations than this package's kernels and may not fit next to the
        # unsharded optimizer state at the main arm's micro-batch: it then runs the same global batch in micro-batches
        # of half the size (recorded in `micro_batch_per_gpu`)
        tries = [main_mb] + ([main_mb // 2] if world == 1 and main_mb >= 2 else [])
        for b_mb in tries:
            try:
                b = run_arm(kind, b_mb, side_steps, False, False)
                baseline = {"what": ("same model, batch and sharded optimizer with NCCL reduce-scatter / all-gather "
                                     "instead of the fused peer-memory kernels" if world > 1 else
                                     "same model, batch and optimizer with stock PyTorch ops (cuBLAS linear, library "
                                     "fused attention, unfused element-wise ops) instead of this package's kernels"),
                            "value": tps(b["ms_per_step"]), "ms_per_step": b["ms_per_step"], "steps": side_steps,
                            "micro_batch_per_gpu": b_mb, "peak_mem_gib": b["peak_mem_gib"]}
                break
            except Exception as e:  # an out-of-memory baseline must not lose the main number
                baseline = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
                if world > 1:
                    raise
            gc.collect()
            torch.cuda.empty_cache()
    same_mb = None
    if "same_mb" in arms and world > 1 and main_mb != 2 and seqs % 2 == 0:
        try:
            m2 = run_arm(main_kind, 2, side_steps, False, False)
            same_mb = {"value": tps(m2["ms_per_step"]), "ms_per_step": m2["ms_per_step"], "micro_batch_per_gpu": 2,
                       "grad_accum": seqs // 2, "steps": side_steps}
        except Exception as e:
            same_mb = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
            if world > 1:
                raise
    elif main_mb == 2:
        same_mb = {"value": value, "ms_per_step": main["ms_per_step"], "micro_batch_per_gpu": 2,
                   "grad_accum": seqs // 2, "steps": args.steps}

    if rank == 0:
        e2e = None
        if main.get("e2e"):
            e2e = dict(main["e2e"], value=tps(main["e2e"]["ms_per_step"]), unit="tokens/s")
        par = {"single": "single", "zero2": f"fsdp{world} (zero2: fused reduce-scatter+AdamW, overlapped all-gather)",
               "zero2-nccl": f"fsdp{world} (zero2 over NCCL)",
               "zero3": f"fsdp{world} (zero3: weight all-gather and wgrad reduce-scatter inside the GEMMs)"}[main_kind]
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / baseline["value"]) if baseline and "value" in baseline else None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
            "config": {"model": args.model if not args.layers else f"{args.model}[{args.layers} layers]",
                       "global_batch": seqs * world, "seq_len": args.seq_len,
                       "micro_batch_per_gpu": main["micro_batch"], "grad_accum": main["grad_accum"],
                       "parallelism": par,
                       "optimizer": "AdamW lr 2e-5, fp32 master+moments, clip 1.0",
                       "loss_mask": f"positions >= {PROMPT_LEN}",
                       "l2": "no flush: each step streams >100 GB of weights/optimizer state (>> 126 MB L2)"},
            "clocks": main["clocks"], "e2e": e2e, "gpu_launches": main["launches"],
            "impl": "ours" if main_kind != "zero2-nccl" else "ours-nccl-baseline",
            "baseline": baseline, "same_microbatch": same_mb,
            "same_microbatch_value": same_mb.get("value") if same_mb else None,
            "peak_mem_gib": main["peak_mem_gib"],
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
