"""Worker of the tensor-parallel decode test: the paged engine on a model sliced over 2 ranks against the same engine
on the whole model (greedy, and sampled with one seed). Launched by torch.distributed.run with one rank per GPU."""
import datetime
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class Tok:
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
    out_path = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=120))
    dev = torch.device("cuda", torch.cuda.current_device())
    from tunix_b200 import _lib
    from tunix_b200.common.configs import CacheConfig
    from tunix_b200.generate.engine import PagedEngine
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.parallel import tp as tp_lib
    cfg = ModelConfig(family="qwen3", num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=4, head_dim=64,
                      num_kv_heads=2, qk_norm=True, dtype=torch.bfloat16, max_position=512)
    cc = CacheConfig(cache_size=256, num_layers=2, num_kv_heads=2, head_dim=64)
    prompts = [[1, 5, 9, 77, 30], [1, 200, 3], [1] + list(range(10, 40)), [1, 8], [1, 44, 45, 46, 47, 48, 49]]
    whole = create_model(cfg, device=dev, seed=0)
    ref_eng = PagedEngine(whole, Tok(), cc, page_size=16, max_running_requests=3, check_every=4)
    ref = ref_eng(prompt_token_ids=prompts, max_generation_steps=24, return_logprobs=True, eos_tokens=[2])
    ref_s = ref_eng(prompt_token_ids=prompts, max_generation_steps=16, temperature=1.0, seed=7, return_logprobs=True, eos_tokens=[2])
    sliced = create_model(cfg, device=dev, seed=0)
    tp_lib.apply_tensor_parallel(sliced, tp_lib.TPContext(device=dev))
    res = {"rank": rank}
    for graph in (False, True):
        eng = PagedEngine(sliced, Tok(), cc, page_size=16, max_running_requests=3, use_cuda_graph=graph, check_every=4)
        assert eng.tpw == world and eng.n_kv == 1
        got = eng(prompt_token_ids=prompts, max_generation_steps=24, return_logprobs=True, eos_tokens=[2])
        _lib.raise_if_kernel_error()
        agree = total = 0
        first_lp = 0.0
        for a, b, la, lb in zip(ref.tokens, got.tokens, ref.logprobs, got.logprobs):
            n = min(len(a), len(b))
            agree += int((np.asarray(a[:n]) == np.asarray(b[:n])).sum())
            total += n
            first_lp = max(first_lp, abs(float(la[0]) - float(lb[0])))
        res[f"agree_graph{int(graph)}"] = agree / max(total, 1)
        res[f"first_lp_graph{int(graph)}"] = first_lp
        got_s = eng(prompt_token_ids=prompts, max_generation_steps=16, temperature=1.0, seed=7, return_logprobs=True, eos_tokens=[2])
        # every rank of the group must have sampled the same tokens (same logits, same seed)
        flat = torch.tensor([t for row in got_s.tokens for t in row][:64] + [0] * 64, device=dev)[:64]
        others = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(others, flat)
        res[f"ranks_equal_graph{int(graph)}"] = bool(all(torch.equal(o, others[0]) for o in others))
        same = tot = 0
        for a, b in zip(ref_s.tokens, got_s.tokens):
            n = min(len(a), len(b))
            same += int((np.asarray(a[:n]) == np.asarray(b[:n])).sum())
            tot += n
        res[f"sampled_agree_graph{int(graph)}"] = same / max(tot, 1)
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(gathered, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
