"""Paged engine (paged KV, CUDA-graphed decode) against the dense-cache Sampler, and kernel-level checks."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


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


def _model(**kw):
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    base = dict(family="qwen3", num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=4, head_dim=64,
                num_kv_heads=2, qk_norm=True, dtype=torch.bfloat16, max_position=512)
    base.update(kw)
    return create_model(ModelConfig(**base), device=torch.device("cuda"), seed=0)


def test_paged_decode_kernel_matches_reference():
    from tunix_b200.ops import kernels as K
    torch.manual_seed(0)
    B, N, KH, H, page, max_pages = 5, 8, 2, 128, 16, 40
    lens = torch.tensor([1, 17, 300, 600, 255], device="cuda", dtype=torch.int32)
    num_pages = B * max_pages
    kp = torch.randn(num_pages, page, KH * H, device="cuda", dtype=torch.bfloat16)
    vp = torch.randn_like(kp)
    perm = torch.randperm(num_pages, device="cuda").int().view(B, max_pages)
    q = torch.randn(B, N, H, device="cuda", dtype=torch.bfloat16)
    slots = torch.arange(B, device="cuda", dtype=torch.int32)
    out = K.paged_decode(q, kp, vp, perm, slots, lens, num_kv_heads=KH, page_size=page, max_ctx=640, scale=1 / math.sqrt(H))
    for b in range(B):
        L = int(lens[b])
        idx = torch.arange(L, device="cuda")
        rows = perm[b][idx // page].long() * page + idx % page
        k = kp.view(-1, KH, H)[rows].float()
        v = vp.view(-1, KH, H)[rows].float()
        kk = k.repeat_interleave(N // KH, dim=1)
        vv = v.repeat_interleave(N // KH, dim=1)
        s = torch.einsum("nh,lnh->nl", q[b].float(), kk) / math.sqrt(H)
        ref = torch.einsum("nl,lnh->nh", torch.softmax(s, -1), vv)
        assert torch.allclose(out[b].float(), ref, atol=2e-2, rtol=2e-2), b


@pytest.mark.parametrize("M,N,K_", [(8, 4096, 512), (64, 1024, 4096), (100, 12288, 256)])
def test_small_m_gemm_tiles(M, N, K_):
    from tunix_b200 import _lib
    from tunix_b200.ops import kernels as K
    torch.manual_seed(1)
    A = torch.randn(M, K_, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K_, device="cuda", dtype=torch.bfloat16)
    out = K.gemm(A, B, out_dtype=torch.float32)
    _lib.raise_if_kernel_error()
    ref = A.float() @ B.float().t()
    assert ((out - ref).norm() / ref.norm()).item() < 2e-3


@pytest.mark.parametrize("graph", [False, True])
def test_engine_matches_dense_sampler_greedy(graph):
    from tunix_b200 import _lib
    from tunix_b200.common.configs import CacheConfig
    from tunix_b200.generate.engine import PagedEngine
    from tunix_b200.generate.sampler import Sampler
    model = _model()
    cc = CacheConfig(cache_size=256, num_layers=2, num_kv_heads=2, head_dim=64)
    prompts = [[1, 5, 9, 77, 30], [1, 200, 3], [1] + list(range(10, 40)), [1, 8]]
    dense = Sampler(model, Tok(), cc)(prompt_token_ids=prompts, max_generation_steps=24, return_logprobs=True, eos_tokens=[2])
    eng = PagedEngine(model, Tok(), cc, page_size=16, max_running_requests=3, use_cuda_graph=graph, check_every=4)
    paged = eng(prompt_token_ids=prompts, max_generation_steps=24, return_logprobs=True, eos_tokens=[2])
    _lib.raise_if_kernel_error()
    agree = 0
    for a, b, la, lb in zip(dense.tokens, paged.tokens, dense.logprobs, paged.logprobs):
        n = min(len(a), len(b))
        same = int((np.asarray(a[:n]) == np.asarray(b[:n])).sum())
        agree += same
        # log-probs of the first token come from identical prefill math
        assert abs(la[0] - lb[0]) < 5e-2
    total = sum(min(len(a), len(b)) for a, b in zip(dense.tokens, paged.tokens))
    assert agree / total > 0.9, (agree, total)       # bf16 near-ties may flip an argmax late in a sequence


def test_engine_sampling_reproducible_and_wave_independent():
    from tunix_b200.common.configs import CacheConfig
    from tunix_b200.generate.engine import PagedEngine
    model = _model()
    cc = CacheConfig(cache_size=128, num_layers=2, num_kv_heads=2, head_dim=64)
    eng = PagedEngine(model, Tok(), cc, page_size=16, max_running_requests=4)
    p = [[1, 4, 5, 6], [1, 9, 9], [1, 7], [1, 3, 3, 3, 3]]
    a = eng(prompt_token_ids=p, max_generation_steps=12, temperature=1.0, top_p=0.95, seed=5, return_logprobs=True, eos_tokens=[2])
    b = eng(prompt_token_ids=p, max_generation_steps=12, temperature=1.0, top_p=0.95, seed=5, return_logprobs=True, eos_tokens=[2])
    c = eng(prompt_token_ids=p, max_generation_steps=12, temperature=1.0, top_p=0.95, seed=6, return_logprobs=True, eos_tokens=[2])
    assert all(np.array_equal(x, y) for x, y in zip(a.tokens, b.tokens))
    assert any(not np.array_equal(x, y) for x, y in zip(a.tokens, c.tokens))
    assert eng.pool.free_pages == eng.pool.num_pages
