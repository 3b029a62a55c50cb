"""Plain-PyTorch restatements of every op (fp32-friendly, differentiable by autograd).

These are the CPU path (small configs, unit tests, gloo ranks) and the numerical
oracle for the CUDA kernels. They state the math of the reference implementation:
RMSNorm (tunix/models/llama3/model.py:290-297, gemma `(1+w)` tunix/models/gemma/model.py:730-740),
half-split RoPE (llama3/model.py:249-270), GQA attention with causal / sliding-window /
segment masks and tanh soft-cap (gemma/model.py:442-483), SwiGLU / GeGLU
(llama3/model.py:489-496, gemma/model.py:592-601) and the lm_head log-probabilities
(tunix/rl/common.py:207-226).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

MASK_VALUE = -2.3819763e38  # large negative used by the reference instead of -inf


def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float, add_one: bool = False) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + (1.0 if add_one else 0.0)
    return (xf * rstd * wf).to(x.dtype)


def rope_tables(head_dim: int, max_pos: int, theta: float, scale_factor: float = 1.0,
                device=None, llama3_scaling: dict | None = None):
    """cos/sin tables [max_pos, head_dim/2] in fp32 (computed in fp64 for accuracy)."""
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64, device=device) * 2.0 / head_dim))
    if llama3_scaling:
        factor = llama3_scaling.get("factor", 8.0)
        lo = llama3_scaling.get("low_freq_factor", 1.0)
        hi = llama3_scaling.get("high_freq_factor", 4.0)
        old = llama3_scaling.get("original_max_position_embeddings", 8192)
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor,
                             torch.where(wavelen < old / hi, inv, (1 - smooth) * inv / factor + smooth * inv))
        inv = scaled
    pos = torch.arange(max_pos, dtype=torch.float64, device=device)
    ang = pos[:, None] * inv[None, :] / scale_factor
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


def rope_ref(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [..., T, heads, H]; positions [..., T] (int); half-split rotation."""
    H = x.shape[-1]
    c = cos[positions.long()].unsqueeze(-2)
    s = sin[positions.long()].unsqueeze(-2)
    xf = x.float()
    x1, x2 = xf[..., : H // 2], xf[..., H // 2:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def build_attention_mask(Tq: int, Tk: int, *, causal: bool, window: int, q_off: int | None,
                         seg_q=None, seg_k=None, device=None) -> torch.Tensor:
    """Boolean [B or 1, 1, Tq, Tk] mask, True = attend."""
    if q_off is None:
        q_off = Tk - Tq
    qpos = torch.arange(Tq, device=device)[:, None] + q_off
    kpos = torch.arange(Tk, device=device)[None, :]
    m = torch.ones(Tq, Tk, dtype=torch.bool, device=device)
    if causal:
        m &= kpos <= qpos
    if window and window > 0:
        m &= kpos > qpos - window
    m = m[None, None]
    if seg_q is not None and seg_k is not None:
        m = m & (seg_q[:, None, :, None] == seg_k[:, None, None, :])
    return m


def attention_ref(q, k, v, *, scale: float, causal: bool = True, window: int = 0, softcap: float = 0.0,
                  q_off: int | None = None, seg_q=None, seg_k=None, mask: torch.Tensor | None = None):
    """q [B,Tq,N,H], k/v [B,Tk,KH,H] -> [B,Tq,N,H]. fp32 softmax. `mask` (bool, True=attend) overrides."""
    B, Tq, N, H = q.shape
    Tk, KH = k.shape[1], k.shape[2]
    G = N // KH
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    if G > 1:
        kf = kf.repeat_interleave(G, dim=1)
        vf = vf.repeat_interleave(G, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if softcap and softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    if mask is None:
        mask = build_attention_mask(Tq, Tk, causal=causal, window=window, q_off=q_off, seg_q=seg_q, seg_k=seg_k,
                                    device=q.device)
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3).to(q.dtype)


def glu_ref(g: torch.Tensor, u: torch.Tensor, kind: str) -> torch.Tensor:
    gf = g.float()
    act = F.silu(gf) if kind == "silu" else F.gelu(gf, approximate="tanh")
    return (act * u.float()).to(g.dtype)


def lm_head_logprobs_ref(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, *, softcap: float = 0.0,
                         temperature: float = 1.0, want_entropy: bool = False, chunk: int = 0):
    """Per-token log p(target) (and entropy) of logits = h @ w^T, fp32, optionally in row chunks.

    h [rows, D], w [V, D], targets [rows] (negative = ignore -> logp 0).
    """
    rows = h.shape[0]
    step = chunk if chunk and chunk > 0 else rows
    lps, ents = [], []
    for s0 in range(0, max(rows, 1), max(step, 1)):
        hc = h[s0:s0 + step]
        if hc.shape[0] == 0:
            break
        z = hc.float() @ w.float().t()
        if softcap and softcap > 0:
            z = softcap * torch.tanh(z / softcap)
        z = z / temperature
        lsm = torch.log_softmax(z, dim=-1)
        tg = targets[s0:s0 + step].long()
        valid = (tg >= 0) & (tg < w.shape[0])
        lp = lsm.gather(1, tg.clamp(0, w.shape[0] - 1)[:, None])[:, 0] * valid
        lps.append(lp)
        if want_entropy:
            ents.append(-(lsm.exp() * lsm).sum(-1))
    logp = torch.cat(lps) if lps else h.new_zeros((0,), dtype=torch.float32)
    ent = (torch.cat(ents) if ents else None) if want_entropy else None
    return logp, ent


def topk_router_ref(logits: torch.Tensor, k: int, renormalize: bool = True):
    """softmax -> top-k -> renormalise (tunix/models/qwen3/model.py:895-902)."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, idx, probs
