"""Numerics of the sm_100a kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _k():
    from tunix_b200.ops import kernels
    return kernels


def _check_status():
    from tunix_b200 import _lib
    _lib.raise_if_kernel_error()


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 128), (384, 1024, 4096), (200, 264, 72),
                                   (1000, 136, 520), (4096, 4096, 1024)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    k = _k()
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = k.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    _check_status()
    assert _rel_err(out, ref) < 1e-2
    out32 = k.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    _check_status()
    assert _rel_err(out32, ref) < 2e-3


def test_gemm_epilogues():
    k = _k()
    torch.manual_seed(1)
    M, N, K = 512, 768, 256
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    ref = 0.5 * (A.float() @ B.float().t()) + bias.float() + res.float()
    out = k.gemm(A, B, bias=bias, residual=res, alpha=0.5)
    assert _rel_err(out, ref) < 1e-2
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    k.gemm(A, B, out=acc, accumulate=True)
    assert _rel_err(acc, A.float() @ B.float().t() + 1.0) < 2e-3
    # strided output: write into the right half of a wider buffer
    wide = torch.zeros(M, 2 * N, device="cuda", dtype=torch.bfloat16)
    k.gemm(A, B, out=wide[:, N:])
    assert _rel_err(wide[:, N:], A.float() @ B.float().t()) < 1e-2
    assert wide[:, :N].abs().max().item() == 0
    _check_status()


@pytest.mark.parametrize("rows,D,add_one", [(37, 256, False), (1024, 4096, False), (300, 3584, True), (4096, 128, False),
                                             (64, 8192, False), (5, 1536, True)])
def test_rmsnorm(rows, D, add_one):
    k = _k()
    torch.manual_seed(2)
    x = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(D, device="cuda") * 0.1 + (0.0 if add_one else 1.0)).to(torch.bfloat16)
    dy = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    rstd_ref = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)
    yref = xf * rstd_ref * (wf + (1.0 if add_one else 0.0))
    yref.backward(dy.float())
    y, rstd = k.rmsnorm_fwd(x, w, 1e-6, add_one)
    assert _rel_err(y, yref) < 1e-2
    dx, dw = k.rmsnorm_bwd(dy, x, w, rstd, add_one)
    assert _rel_err(dx, xf.grad) < 1e-2
    assert _rel_err(dw, wf.grad) < 1e-2


def test_rope_roundtrip_and_reference():
    k = _k()
    torch.manual_seed(3)
    tokens, heads, H = 513, 6, 128
    x = torch.randn(tokens, heads, H, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 2048, (tokens,), device="cuda", dtype=torch.int32)
    inv = 1.0 / (10000.0 ** (torch.arange(0, H // 2, device="cuda", dtype=torch.float64) * 2 / H))
    ang = torch.arange(2048, device="cuda", dtype=torch.float64)[:, None] * inv[None]
    cos, sin = ang.cos().float().contiguous(), ang.sin().float().contiguous()
    xf = x.float()
    c = cos[pos.long()][:, None, :]
    s = sin[pos.long()][:, None, :]
    x1, x2 = xf[..., : H // 2], xf[..., H // 2:]
    ref = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    y = k.rope_(x.clone(), pos, cos, sin)
    assert _rel_err(y, ref) < 1e-2
    back = k.rope_(y.clone(), pos, cos, sin, backward=True)
    assert _rel_err(back, x) < 2e-2


@pytest.mark.parametrize("kind", [0, 1])
def test_glu(kind):
    k = _k()
    torch.manual_seed(4)
    rows, F = 333, 1024
    g = torch.randn(rows, F, device="cuda", dtype=torch.bfloat16)
    u = torch.randn(rows, F, device="cuda", dtype=torch.bfloat16)
    dh = torch.randn(rows, F, device="cuda", dtype=torch.bfloat16)
    gf, uf = g.float().requires_grad_(True), u.float().requires_grad_(True)
    act = torch.nn.functional.silu(gf) if kind == 0 else torch.nn.functional.gelu(gf, approximate="tanh")
    href = act * uf
    href.backward(dh.float())
    h = k.glu_fwd(g, u, kind)
    assert _rel_err(h, href) < 1e-2
    dg, du = k.glu_bwd(dh, g, u, kind)
    assert _rel_err(dg, gf.grad) < 1.5e-2
    assert _rel_err(du, uf.grad) < 1.5e-2


def test_embedding():
    k = _k()
    torch.manual_seed(5)
    V, D, T = 1000, 256, 777
    table = torch.randn(V, D, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    out = k.embedding_fwd(ids, table, scale=2.0)
    assert _rel_err(out, table[ids.long()].float() * 2.0) < 1e-2
    dout = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    dtable = torch.zeros_like(table)
    k.embedding_bwd(ids, dout, dtable, scale=2.0)
    ref = torch.zeros(V, D, device="cuda").index_add_(0, ids.long(), dout.float() * 2.0)
    assert _rel_err(dtable, ref) < 2e-2


@pytest.mark.parametrize("softcap,temp", [(0.0, 1.0), (30.0, 0.7)])
def test_logsoftmax_and_dlogits(softcap, temp):
    k = _k()
    torch.manual_seed(6)
    rows, V = 65, 5003
    raw = (torch.randn(rows, V, device="cuda") * 4).requires_grad_(True)
    tg = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    tg[3] = -1
    z = raw
    if softcap > 0:
        z = softcap * torch.tanh(z / softcap)
    z = z / temp
    lsm = torch.log_softmax(z, -1)
    logp_ref = lsm.gather(1, tg.clamp(min=0).long()[:, None])[:, 0] * (tg >= 0)
    ent_ref = -(lsm.exp() * lsm).sum(-1)
    gl = torch.randn(rows, device="cuda")
    ge = torch.randn(rows, device="cuda")
    ((logp_ref * gl).sum() + (ent_ref * ge).sum()).backward()
    logp, lse, ent = k.logsoftmax_gather(raw.detach(), tg, softcap=softcap, temperature=temp, want_entropy=True)
    assert torch.allclose(logp, logp_ref.detach(), atol=2e-3, rtol=1e-3)
    assert torch.allclose(ent, ent_ref.detach(), atol=2e-3, rtol=1e-3)
    d = k.dlogits(raw.detach(), tg, lse, ent, gl, ge, softcap=softcap, temperature=temp)
    assert _rel_err(d, raw.grad) < 1.5e-2


def test_adamw_matches_torch():
    k = _k()
    torch.manual_seed(7)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    p32, m, v = p.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        gs = g * step
        ref_p.grad = gs.clone()
        opt.step()
        k.adamw(p32, m, v, gs.to(torch.bfloat16).float(), p16, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                weight_decay=0.1, step=step)
    # torch applies decay as p *= (1 - lr*wd) before the Adam step; optax adds wd*p to the update.
    # The two differ at O(lr^2 * wd), far below this tolerance.
    assert _rel_err(p32, ref_p.detach()) < 2e-3
    assert _rel_err(p16, p32) < 5e-3
    ss = torch.zeros(1, device="cuda")
    k.sumsq(g, ss)
    assert abs(ss.item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-4


@pytest.mark.parametrize("M,N,K_,a_mn,b_mn", [(2048, 2048, 512, False, False), (4096, 1536, 1024, False, True),
                                              (2304, 2048, 768, True, True), (2000, 2100, 320, False, False),
                                              (8192, 4096, 4096, False, False)])
def test_gemm_cta_pair_tiles(M, N, K_, a_mn, b_mn):
    """Problems with a wave of 256 x 256 tiles run on CTA pairs (tcgen05.mma.cta_group::2): layouts, ragged edges,
    bias / residual / alpha, fp32 accumulation into an existing buffer."""
    k = _k()
    torch.manual_seed(5)
    A = torch.randn((K_, M) if a_mn else (M, K_), device="cuda", dtype=torch.bfloat16)
    B = (torch.randn((K_, N) if b_mn else (N, K_), device="cuda") * 0.05).to(torch.bfloat16)
    ref = (A.float().t() if a_mn else A.float()) @ (B.float() if b_mn else B.float().t())
    out = k.gemm(A, B, a_mn=a_mn, b_mn=b_mn)
    _check_status()
    assert _rel_err(out, ref) < 5e-3
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out2 = k.gemm(A, B, a_mn=a_mn, b_mn=b_mn, bias=bias, residual=res, alpha=0.25)
    _check_status()
    assert _rel_err(out2, 0.25 * ref + bias.float() + res.float()) < 5e-3
    acc = torch.full((M, N), 2.0, device="cuda", dtype=torch.float32)
    k.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True)
    _check_status()
    assert _rel_err(acc, ref + 2.0) < 2e-3


@pytest.mark.parametrize("shape,block", [((256, 512), 64), ((100, 72), 32), ((3, 50), 64)])
def test_nf4_dequant_kernel_matches_reference(shape, block):
    from tunix_b200.lora import NF4Weight
    torch.manual_seed(3)
    w = torch.randn(*shape, device="cuda", dtype=torch.bfloat16)
    q = NF4Weight(w, block)
    got = q.dequantize()
    _check_status()
    cpu = NF4Weight(w.cpu(), block).dequantize()
    assert got.shape == w.shape and torch.allclose(got.float().cpu(), cpu.float(), atol=1e-2, rtol=1e-2)
    assert (got.float() - w.float()).abs().mean() < 0.15


@pytest.mark.parametrize("rows,V,D,softcap,temp", [(512, 5000, 256, 0.0, 1.0), (1024, 33000, 512, 30.0, 0.7), (300, 128256, 128, 0.0, 1.0)])
def test_fused_lm_head_logprobs_match_reference(rows, V, D, softcap, temp):
    """The log-softmax epilogue of the two-SM GEMM (no logits in memory) against fp32 PyTorch, forward and backward."""
    from tunix_b200.ops import functional as F
    torch.manual_seed(9)
    h = (torch.randn(rows, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(V, D, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    tg = torch.randint(0, V, (rows,), device="cuda")
    tg[::17] = -1                                                  # ignored positions
    logp, ent = F.lm_head_logprobs(h, w, tg, softcap=softcap, temperature=temp, want_entropy=True)
    _check_status()
    z = h.detach().float() @ w.detach().float().t()
    if softcap:
        z = softcap * torch.tanh(z / softcap)
    z = z / temp
    ref_lp = torch.log_softmax(z, -1).gather(-1, tg.clamp(min=0)[:, None]).squeeze(-1)
    ref_lp = torch.where(tg >= 0, ref_lp, torch.zeros_like(ref_lp))
    p = torch.softmax(z, -1)
    ref_ent = -(p * torch.log_softmax(z, -1)).sum(-1)
    assert torch.allclose(logp, ref_lp, atol=3e-2, rtol=2e-2), float((logp - ref_lp).abs().max())
    assert torch.allclose(ent, ref_ent, atol=3e-2, rtol=2e-2)
    g = torch.randn(rows, device="cuda")
    g2 = torch.randn(rows, device="cuda") * 0.3
    ((logp * g).sum() + (ent * g2).sum()).backward()          # both gradient terms of the fused epilogue
    _check_status()
    hr = h.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    zr = hr @ wr.t()
    if softcap:
        zr = softcap * torch.tanh(zr / softcap)
    lsm = torch.log_softmax(zr / temp, -1)
    lp2 = lsm.gather(-1, tg.clamp(min=0)[:, None]).squeeze(-1)
    ent2 = -(lsm.exp() * lsm).sum(-1)
    ((torch.where(tg >= 0, lp2, torch.zeros_like(lp2)) * g).sum() + (ent2 * g2).sum()).backward()
    assert _rel_err(h.grad, hr.grad) < 3e-2 and _rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("M,N,K,r", [(2048, 4096, 1024, 16), (2304, 2560, 520, 8), (4096, 2048, 2048, 64), (2048, 4096, 512, 72),
                                     (128, 256, 64, 16)])
@pytest.mark.parametrize("b_mn", [False, True])
def test_gemm_with_second_segment(M, N, K, r, b_mn):
    """A @ B^T + A2 @ B2^T in one launch (adapter rank r as extra k-blocks; the last shape falls back to two GEMMs)."""
    k = _k()
    torch.manual_seed(11)
    A = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    A2 = torch.randn(M, r, device="cuda", dtype=torch.bfloat16)
    B2 = torch.randn(N, r, device="cuda", dtype=torch.bfloat16) * 4
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t() + A2.float() @ B2.float().t()
    b, b2 = (B.t().contiguous(), B2.t().contiguous()) if b_mn else (B, B2)
    out = k.gemm_ext(A, b, A2, b2, b_mn=b_mn)
    _check_status()
    assert _rel_err(out, ref) < 1e-2
    # the low-rank part alone must be right too (it is small next to the main product)
    low = out.float() - (A.float() @ B.float().t())
    assert _rel_err(low, A2.float() @ B2.float().t()) < 0.2
    out = k.gemm_ext(A, b, A2, b2, b_mn=b_mn, bias=bias, residual=res)
    _check_status()
    full = ref + bias.float() + res.float()
    assert _rel_err(out, full) < 1e-2
    assert torch.allclose(out.float(), full, atol=0.02 * full.abs().max().item(), rtol=2e-2)


@pytest.mark.parametrize("with_bias,with_res", [(False, False), (True, True)])
def test_lora_linear_matches_fp32(with_bias, with_res):
    """Fused LoRA projection (forward, input gradient, adapter gradients) against fp32 PyTorch."""
    from tunix_b200.ops import functional as F
    torch.manual_seed(5)
    M, D, O, r, s = 2048, 1024, 3072, 16, 2.0
    x = (torch.randn(4, M // 4, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(O, D, device="cuda") * 0.05).to(torch.bfloat16)
    a = (torch.randn(r, D, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    b = (torch.randn(O, r, device="cuda") * 0.2).to(torch.bfloat16).requires_grad_()
    bias = (torch.randn(O, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_() if with_bias else None
    res = (torch.randn(4, M // 4, O, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_() if with_res else None
    y = F.lora_linear(x, w, bias, a, b, s, res)
    g = torch.randn_like(y)
    y.backward(g)
    _check_status()
    xf, af, bf = (t.detach().float().requires_grad_() for t in (x, a, b))
    yf = xf @ w.float().t() + s * (xf @ af.t()) @ bf.t()
    if with_bias:
        yf = yf + bias.detach().float()
    if with_res:
        yf = yf + res.detach().float()
    yf.backward(g.float())
    assert _rel_err(y, yf) < 1e-2
    assert _rel_err(x.grad, xf.grad) < 1e-2
    assert _rel_err(a.grad, af.grad) < 2e-2
    assert _rel_err(b.grad, bf.grad) < 2e-2
    if with_res:
        assert torch.equal(res.grad, g)
    if with_bias:
        assert _rel_err(bias.grad, g.float().sum((0, 1))) < 1e-2


def test_qlora_linear_keeps_no_expanded_weight():
    """A LoRA projection over an NF4 base: same values and gradients as the projection over the expanded weight, and
    between forward and backward nothing of the size of the expanded weight stays allocated."""
    from tunix_b200 import lora
    from tunix_b200.models.transformer import Linear
    torch.manual_seed(2)
    D, O = 2048, 4096
    lin = Linear(D, O, dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        lin.weight.normal_(0, 0.05)

    class _M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = lin

    m = _M()
    lora.apply_lora_to_model(m, lora.LoraProvider(rank=16, alpha=32.0, weight_qtype="nf4", module_path=".*proj"))
    with torch.no_grad():
        lin.lora_b.normal_(0, 0.05)
    w_full = lin.quant.dequantize().float()
    x = (torch.randn(2, 1024, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    y = lin(x)                                   # first call allocates the shared scratch
    del y
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    y = lin(x)
    torch.cuda.synchronize()
    held = torch.cuda.memory_allocated() - before
    weight_bytes = D * O * 2
    # y itself (2 * 1024 * O * 2 bytes) plus the rank-16 intermediate, but no [O, D] bf16 tensor
    assert held < 2 * 1024 * O * 2 + weight_bytes // 4, (held, weight_bytes)
    g = torch.randn_like(y)
    y.backward(g)
    _check_status()
    xf = x.detach().float().requires_grad_()
    af, bf = lin.lora_a.detach().float().requires_grad_(), lin.lora_b.detach().float().requires_grad_()
    yf = xf @ w_full.t() + lin.lora_scale * (xf @ af.t()) @ bf.t()
    yf.backward(g.float())
    assert _rel_err(y, yf) < 1e-2 and _rel_err(x.grad, xf.grad) < 1e-2
    assert _rel_err(lin.lora_a.grad, af.grad) < 2e-2 and _rel_err(lin.lora_b.grad, bf.grad) < 2e-2


@pytest.mark.parametrize("M,F,D,kind", [(64, 12288, 1024, "silu"), (16, 1408, 512, "gelu"), (200, 2816, 256, "silu"), (256, 4096, 512, "silu")])
def test_packed_gemm_with_gated_epilogue(M, F, D, kind):
    """Fused gate / up projection on a pre-tiled, row-interleaved weight with act(gate) * up in the epilogue."""
    k = _k()
    torch.manual_seed(4)
    x = (torch.randn(M, D, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(2 * F, D, device="cuda") * 0.05).to(torch.bfloat16)
    pw = k.PackedWeight(w, glu=True)
    out = k.gemm_packed(x, pw, glu=k.GLU_SILU if kind == "silu" else k.GLU_GELU)
    _check_status()
    z = x.float() @ w.float().t()
    g, u = z[:, :F], z[:, F:]
    act = torch.nn.functional.silu(g) if kind == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    ref = act * u
    assert out.shape == (M, F)
    assert _rel_err(out, ref) < 1e-2
    assert torch.allclose(out.float(), ref, atol=0.02 * ref.abs().max().item() + 1e-3, rtol=3e-2)
