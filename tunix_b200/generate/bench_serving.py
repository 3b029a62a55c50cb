"""Serving benchmark: `python -m tunix_b200.generate.bench_serving [--model qwen3_8b] [--layers 8] [--requests 256]`

The same set of requests (random prompt ids of mixed length, mixed token limits, no EOS) is served twice by one
`EngineServer` over the paged engine: submitted directly from threads, then through the OpenAI-style HTTP front end
on the loop-back interface with `--clients` concurrent connections. Prints one JSON line with both throughputs
(generated tokens per second of wall-clock, from the first submission to the last answer) and the request latency
percentiles over HTTP. Random-init weights; the ids a prompt decodes to are irrelevant to the timing."""
from __future__ import annotations

import argparse
import json
import sys
import time
import urllib.request
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch


class _Tok:
    """One token per character so that a prompt of n characters is n ids; no id ends a sequence."""

    def encode(self, s):
        return [3 + (ord(c) % 997) for c in s]

    def decode(self, ids):
        return "".join(chr(97 + int(i) % 26) for i in ids)

    def bos_id(self):
        return 1

    def eos_id(self):
        return -1

    def pad_id(self):
        return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3_8b")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = preset)")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--clients", type=int, default=128)
    ap.add_argument("--max-running", type=int, default=128)
    ap.add_argument("--prompt", type=int, default=256, help="longest prompt; lengths are uniform in [prompt/4, prompt]")
    ap.add_argument("--gen", type=int, default=256, help="largest token limit; limits are uniform in [gen/4, gen]")
    ap.add_argument("--check-every", type=int, default=8)
    a = ap.parse_args(argv)
    from tunix_b200.common.configs import CacheConfig
    from tunix_b200.generate.engine import EngineServer, PagedEngine
    from tunix_b200.generate.openai_server import serve
    from tunix_b200.models.config import get_config
    from tunix_b200.models.transformer import create_model
    dev = torch.device("cuda")
    cfg = get_config(a.model).replace(dtype=torch.bfloat16, max_position=a.prompt + a.gen + 8)
    if a.layers:
        cfg = cfg.replace(num_layers=a.layers)
    model = create_model(cfg, device=dev, seed=0)
    tok = _Tok()
    engine = PagedEngine(model, tok, CacheConfig(a.prompt + a.gen + 8, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim), page_size=64,
                         max_running_requests=a.max_running, check_every=a.check_every)
    rng = np.random.default_rng(0)
    lens = rng.integers(a.prompt // 4, a.prompt + 1, a.requests)
    limits = rng.integers(a.gen // 4, a.gen + 1, a.requests).tolist()
    texts = ["".join(chr(97 + int(c)) for c in rng.integers(0, 26, int(n))) for n in lens]
    prompts = [tok.encode(t) for t in texts]
    out = {"model": a.model, "layers": cfg.num_layers, "requests": a.requests, "clients": a.clients, "max_running": a.max_running}
    with EngineServer(engine, max_new_tokens=a.gen, max_prompt_length=a.prompt, temperature=1.0, seed=1, eos_tokens=[-1]) as srv:
        with ThreadPoolExecutor(a.clients) as pool:
            list(pool.map(lambda i: srv.generate(prompts[i], 8), range(min(a.max_running, a.requests))))      # warm-up: graphs, pages
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = list(pool.map(lambda i: srv.generate(prompts[i], limits[i]), range(a.requests)))
            dt = time.perf_counter() - t0
        n = sum(len(t) for t, _ in res)
        out["direct"] = {"tokens": n, "seconds": round(dt, 3), "tokens_per_s": round(n / dt, 1)}
        with serve(srv, tok, model_name=a.model) as http:
            def call(i):
                body = json.dumps({"prompt": texts[i], "max_tokens": limits[i]}).encode()
                t = time.perf_counter()
                with urllib.request.urlopen(urllib.request.Request(http.url + "/v1/completions", data=body), timeout=600) as r:
                    ans = json.loads(r.read())
                return ans["usage"]["completion_tokens"], time.perf_counter() - t
            with ThreadPoolExecutor(a.clients) as pool:
                list(pool.map(call, range(min(16, a.requests))))
                t0 = time.perf_counter()
                res = list(pool.map(call, range(a.requests)))
                dt = time.perf_counter() - t0
        n = sum(r[0] for r in res)
        lat = np.sort(np.array([r[1] for r in res]))
        out["http"] = {"tokens": n, "seconds": round(dt, 3), "tokens_per_s": round(n / dt, 1),
                       "latency_s": {"p50": round(float(lat[len(lat) // 2]), 3), "p90": round(float(lat[int(len(lat) * 0.9)]), 3),
                                     "max": round(float(lat[-1]), 3)}}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
