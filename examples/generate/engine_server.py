"""Serving single requests from many threads with the paged engine's server mode.

    python examples/generate/engine_server.py            (one B200; random-init Qwen3-style model, synthetic prompts)

Every `generate` call is one request with its own token limit; requests join the running batch at the next
check point (continuous batching). `pause()` / `resume()` bracket an in-place weight update. With `--http PORT` the
same server is then put behind the OpenAI-style HTTP front end (`/v1/completions`, `/v1/chat/completions`) until
interrupted:

    curl -s 127.0.0.1:8000/v1/completions -d '{"prompt": "hello", "max_tokens": 16}'"""
import argparse
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch

from tunix_b200.common.configs import CacheConfig
from tunix_b200.generate.engine import EngineServer, PagedEngine
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model


class Tok:                      # the engine needs ids for bos / eos / pad and a decoder for the text field
    def encode(self, s):
        return [3 + (ord(c) % 200) for c in s]

    def decode(self, ids):
        return " ".join(str(int(i)) for i in ids)

    def bos_id(self):
        return 1

    def eos_id(self):
        return 2

    def pad_id(self):
        return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--http", type=int, default=None, help="serve the OpenAI-style routes on this port afterwards")
    args = ap.parse_args()
    cfg = ModelConfig(family="qwen3", num_layers=4, vocab_size=4096, embed_dim=1024, hidden_dim=3072, num_heads=8, head_dim=128,
                      num_kv_heads=2, qk_norm=True, dtype=torch.bfloat16, max_position=1024)
    model = create_model(cfg, device=torch.device("cuda"), seed=0)
    engine = PagedEngine(model, Tok(), CacheConfig(1024, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim), page_size=64,
                         max_running_requests=32, check_every=8)
    rng = np.random.default_rng(0)
    prompts = [[1] + rng.integers(3, cfg.vocab_size, int(n)).tolist() for n in rng.integers(8, 200, 96)]
    limits = rng.integers(16, 256, len(prompts)).tolist()
    with EngineServer(engine, max_new_tokens=256, max_prompt_length=256, temperature=1.0, top_p=0.95, seed=1, eos_tokens=[2]) as srv:
        t0 = time.perf_counter()
        with ThreadPoolExecutor(48) as pool:
            outs = list(pool.map(lambda a: srv.generate(a[0], a[1]), zip(prompts, limits)))
        dt = time.perf_counter() - t0
        n = sum(len(t) for t, _ in outs)
        print(f"{len(outs)} requests, {n} tokens in {dt:.2f} s ({n / dt:.0f} tokens/s), {srv.admitted} admitted")
        srv.pause()                                   # nothing is in flight now
        with torch.no_grad():
            for p in model.parameters():
                p.mul_(0.999)                         # stands in for an optimizer step / weight sync
        srv.resume()
        toks, lps = srv.generate(prompts[0], 8)
        print("after the weight update:", toks.tolist(), [round(float(x), 3) for x in lps])
        if args.http is not None:
            from tunix_b200.generate.openai_server import serve
            with serve(srv, Tok(), model_name="qwen3-random-init", port=args.http) as http:
                print("serving on", http.url)
                try:
                    while True:
                        time.sleep(1.0)
                except KeyboardInterrupt:
                    pass


if __name__ == "__main__":
    main()
