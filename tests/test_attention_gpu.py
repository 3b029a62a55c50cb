"""tcgen05 flash attention (forward and backward) against an fp32 PyTorch reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_attention(q, k, v, scale, causal, window, softcap, seg_q, seg_k):
    B, Tq, N, H = q.shape
    Tk, KH = k.shape[1], k.shape[2]
    G = N // KH
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(G, dim=1)
    s = torch.einsum("bnqh,bnkh->bnqk", qf, kf) * scale
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    qpos = torch.arange(Tq, device=q.device)[:, None] + (Tk - Tq)
    kpos = torch.arange(Tk, device=q.device)[None, :]
    mask = torch.ones(Tq, Tk, dtype=torch.bool, device=q.device)
    if causal:
        mask &= kpos <= qpos
    if window > 0:
        mask &= kpos > qpos - window
    mask = mask[None, None].expand(B, 1, Tq, Tk)
    if seg_q is not None:
        mask = mask & (seg_q[:, None, :, None] == seg_k[:, None, None, :])
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.einsum("bnqk,bnkh->bnqh", p, vf)
    return o.permute(0, 2, 1, 3)


CASES = [
    # B, Tq, Tk, N, KH, H, causal, window, softcap, segs
    (1, 128, 128, 1, 1, 128, True, 0, 0.0, False),
    (2, 256, 256, 4, 2, 128, True, 0, 0.0, False),
    (2, 200, 200, 4, 1, 64, True, 0, 0.0, False),
    (1, 512, 512, 4, 2, 128, True, 96, 0.0, False),
    (1, 384, 384, 2, 1, 256, True, 0, 50.0, False),
    (2, 320, 320, 4, 2, 128, True, 0, 0.0, True),
    (1, 64, 320, 4, 4, 128, True, 0, 0.0, False),
    (1, 256, 256, 2, 2, 128, False, 0, 0.0, False),
    (1, 1024, 1024, 8, 2, 128, True, 0, 0.0, False),
    # two query tiles per CTA: ragged last tile, a window narrower than a tile, more keys than queries, segments with a
    # soft-cap, no causal mask
    (1, 448, 448, 2, 1, 128, True, 0, 0.0, False),
    (2, 300, 300, 2, 2, 64, True, 64, 0.0, False),
    (1, 384, 640, 4, 2, 128, True, 0, 0.0, False),
    (1, 512, 512, 2, 1, 128, True, 0, 30.0, True),
    (1, 640, 640, 2, 2, 64, False, 0, 0.0, False),
]


def _make(B, Tq, Tk, N, KH, H, segs):
    torch.manual_seed(0)
    q = torch.randn(B, Tq, N, H, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, Tk, KH, H, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, Tk, KH, H, device="cuda", dtype=torch.bfloat16)
    seg_q = seg_k = None
    if segs:
        cuts = torch.tensor([0, Tk // 3, Tk // 3 + 70, Tk], device="cuda")
        seg_k = torch.bucketize(torch.arange(Tk, device="cuda"), cuts[1:], right=True).int()[None].expand(B, Tk).contiguous() + 1
        seg_q = seg_k[:, Tk - Tq:].contiguous()
    return q, k, v, seg_q, seg_k


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()


def _close(a, b, what=""):
    """Element-wise, next to the norm: a handful of wrong elements cannot hide in a large tensor."""
    a, b = a.float(), b.float()
    tol = 0.03 * b.abs().max().item() + 1e-6
    bad = (a - b).abs() > tol + 0.05 * b.abs()
    assert not bad.any(), (what, int(bad.sum()), (a - b).abs().max().item(), tol)


@pytest.mark.parametrize("two_tile", [False, True])
@pytest.mark.parametrize("case", CASES)
def test_attention_forward(case, two_tile, monkeypatch):
    """Both forward kernels: one 128-row query tile per CTA (the default) and two tiles per CTA (opt-in)."""
    if two_tile and (case[5] > 128 or case[1] <= 128):
        pytest.skip("the two-tile kernel serves head dims up to 128 and more than 128 query rows")
    monkeypatch.setenv("TUNIX_B200_ATTN_TWO_TILE", "1" if two_tile else "0")
    from tunix_b200 import _lib
    from tunix_b200.ops import kernels as k_
    B, Tq, Tk, N, KH, H, causal, window, softcap, segs = case
    q, k, v, seg_q, seg_k = _make(B, Tq, Tk, N, KH, H, segs)
    scale = 1.0 / math.sqrt(H)
    o, lse = k_.attn_fwd(q, k, v, scale=scale, causal=causal, window=window, softcap=softcap, seg_q=seg_q, seg_k=seg_k)
    _lib.raise_if_kernel_error()
    ref = ref_attention(q, k, v, scale, causal, window, softcap, seg_q, seg_k)
    assert _rel(o, ref) < 2e-2, _rel(o, ref)
    _close(o, ref, "o")
    # log-sum-exp of every row that sees at least one key
    s_ = torch.einsum("bqnh,bknh->bnqk", q.float(), k.float().repeat_interleave(N // KH, dim=2)) * scale
    if softcap > 0:
        s_ = softcap * torch.tanh(s_ / softcap)
    qpos = torch.arange(Tq, device="cuda")[:, None] + (Tk - Tq)
    kpos = torch.arange(Tk, device="cuda")[None, :]
    m = torch.ones(Tq, Tk, dtype=torch.bool, device="cuda")
    if causal:
        m &= kpos <= qpos
    if window > 0:
        m &= kpos > qpos - window
    m = m[None, None].expand(B, 1, Tq, Tk)
    if seg_q is not None:
        m = m & (seg_q[:, None, :, None] == seg_k[:, None, None, :])
    want = torch.logsumexp(s_.masked_fill(~m, float("-inf")), dim=-1)
    seen = torch.isfinite(want)
    assert torch.allclose(lse[seen], want[seen], atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("case", CASES)
def test_attention_backward(case):
    from tunix_b200 import _lib
    from tunix_b200.ops import kernels as k_
    B, Tq, Tk, N, KH, H, causal, window, softcap, segs = case
    q, k, v, seg_q, seg_k = _make(B, Tq, Tk, N, KH, H, segs)
    scale = 1.0 / math.sqrt(H)
    do = torch.randn(B, Tq, N, H, device="cuda", dtype=torch.bfloat16)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = ref_attention(qf, kf, vf, scale, causal, window, softcap, seg_q, seg_k)
    ref.backward(do.float())
    o, lse = k_.attn_fwd(q, k, v, scale=scale, causal=causal, window=window, softcap=softcap, seg_q=seg_q, seg_k=seg_k)
    dq, dk, dv = k_.attn_bwd(do, q, k, v, o, lse, scale=scale, causal=causal, window=window, softcap=softcap,
                             seg_q=seg_q, seg_k=seg_k)
    _lib.raise_if_kernel_error()
    assert _rel(dv, vf.grad) < 3e-2, ("dv", _rel(dv, vf.grad))
    assert _rel(dk, kf.grad) < 3e-2, ("dk", _rel(dk, kf.grad))
    assert _rel(dq, qf.grad) < 3e-2, ("dq", _rel(dq, qf.grad))
    _close(dv, vf.grad, "dv")
    _close(dk, kf.grad, "dk")
    _close(dq, qf.grad, "dq")
