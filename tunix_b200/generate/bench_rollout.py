"""Rollout throughput benchmark: `python -m tunix_b200.generate.bench_rollout [--model qwen3_8b] [--seqs 256] ...`

Random-init weights, uniform random prompt token ids, no EOS (every sequence generates the full length), so the
number is decode tokens/s of the engine itself: prompt 256, 768 sampled tokens at temperature 1.0 / top-p 1.0
by default (the GRPO benchmark's rollout shape). Prints one JSON line."""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np
import torch


class _Tok:
    def encode(self, s):
        return [3]

    def decode(self, ids):
        return ""

    def bos_id(self):
        return 1

    def eos_id(self):
        return -1

    def pad_id(self):
        return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3_8b")
    ap.add_argument("--seqs", type=int, default=256)
    ap.add_argument("--prompt", type=int, default=256)
    ap.add_argument("--gen", type=int, default=768)
    ap.add_argument("--max-running", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0, help="override layer count (0 = preset)")
    ap.add_argument("--engine", default="paged", choices=["paged", "dense"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-pack", action="store_true", help="decode GEMMs read the weights in place (no pre-tiled copy)")
    ap.add_argument("--check-every", type=int, default=10 ** 9, help="decode steps between looks at the done flags")
    ap.add_argument("--pdl", action="store_true", help="launch decode kernels with programmatic dependent launch")
    args = ap.parse_args(argv)
    from tunix_b200 import _lib
    from tunix_b200.common.configs import CacheConfig
    from tunix_b200.generate.engine import PagedEngine
    from tunix_b200.generate.sampler import Sampler
    from tunix_b200.models.config import get_config
    from tunix_b200.models.transformer import create_model
    from tunix_b200.ops import kernels
    dev = torch.device("cuda")
    cfg = get_config(args.model).replace(dtype=torch.bfloat16, max_position=args.prompt + args.gen + 8)
    if args.layers:
        cfg = cfg.replace(num_layers=args.layers)
    model = create_model(cfg, device=dev, seed=0)
    cc = CacheConfig(args.prompt + args.gen + 8, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim)
    rng = np.random.default_rng(2)
    prompts = rng.integers(3, cfg.vocab_size, (args.seqs, args.prompt)).tolist()
    if args.engine == "paged":
        eng = PagedEngine(model, _Tok(), cc, page_size=64, max_running_requests=args.max_running,
                          use_cuda_graph=not args.no_graph, check_every=args.check_every, use_pdl=args.pdl,
                          pack_weights=not args.no_pack)
    else:
        eng = Sampler(model, _Tok(), cc)
    kw = dict(prompt_token_ids=prompts, max_generation_steps=args.gen, max_prompt_length=args.prompt, temperature=1.0,
              top_p=1.0, seed=2, return_logprobs=True, eos_tokens=[-1])
    eng(**{**kw, "max_generation_steps": 8, "prompt_token_ids": prompts[: min(args.seqs, args.max_running)]})  # warm-up
    torch.cuda.synchronize()
    l0 = kernels.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    out = eng(**kw)
    e1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    _lib.raise_if_kernel_error()
    n_tok = sum(len(t) for t in out.tokens)
    print(json.dumps({"metric": "rollout_decode_tokens_per_sec", "value": n_tok / wall, "unit": "tokens/s",
                      "device_ms": e0.elapsed_time(e1), "wall_s": wall, "generated_tokens": n_tok, "model": args.model,
                      "layers": cfg.num_layers, "seqs": args.seqs, "prompt": args.prompt, "gen": args.gen,
                      "engine": args.engine, "cuda_graph": not args.no_graph, "pdl": args.pdl, "packed": not args.no_pack,
                      "ms_per_decode_step": 1e3 * wall / (args.gen * max(1, -(-args.seqs // args.max_running))),
                      "native_launches_outside_graph": kernels.launch_count - l0,
                      "peak_mem_gib": torch.cuda.max_memory_allocated() / 2 ** 30}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
