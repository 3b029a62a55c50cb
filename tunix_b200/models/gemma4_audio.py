"""Gemma 4 audio encoder (tunix/models/gemma4/audio.py): a conformer over log-mel frames.

  mel frames [B, T, 128] -> two 3x3 stride-2 convolutions (LayerNorm over channels, ReLU) -> linear
                          -> T/4 frames of `hidden_size`, with the validity mask subsampled alongside
  each layer: half-step feed-forward -> local self-attention -> light convolution -> half-step feed-forward -> norm
  -> output projection (with bias) to `output_proj_dims`; `Gemma4MultimodalEmbedder` then maps the frames into the
     decoder's width exactly as for image soft tokens.

The attention is local: a frame sees itself and the `context_left - 2` frames before it (and fewer than
`context_right` frames after it). Its logits are q·k plus a relative-position term q·R[t - s] (R = a projection of sinusoids of the
distance), soft-capped with tanh; queries carry a learned per-channel scale through a softplus. The reference
evaluates this block by block; here the [T, T] banded form is used, which is the same arithmetic for the few
hundred frames an utterance has. Module names follow the Hugging Face checkpoint so its state dict loads as is.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Sequence

import torch
import torch.nn.functional as TF
from torch import nn

from .gemma4_vision import ClippedLinear
from .transformer import Linear, RMSNorm


@dataclass
class Gemma4AudioConfig:
    hidden_size: int = 1024
    num_layers: int = 12
    num_heads: int = 8
    subsampling_conv_channels: Sequence[int] = (128, 32)
    conv_kernel_size: int = 5
    residual_weight: float = 0.5
    attention_chunk_size: int = 12
    attention_context_left: int = 13
    attention_context_right: int = 0
    attention_logit_cap: float = 50.0
    attention_invalid_logits_value: float = -1.0e9
    use_clipped_linears: bool = True
    norm_eps: float = 1e-6
    gradient_clipping: float = 1e10
    output_proj_dims: int = 1536
    audio_token_id: int = 258881
    dtype: torch.dtype = torch.bfloat16


def _clip(x, limit: float):
    limit = min(limit, torch.finfo(x.dtype).max)
    return torch.clamp(x, -limit, limit)


class _SubsampleLayer(nn.Module):
    def __init__(self, c_in: int, c_out: int, eps: float, dtype, device=None):
        super().__init__()
        self.conv = nn.Conv2d(c_in, c_out, kernel_size=3, stride=2, padding=1, bias=False, dtype=dtype, device=device)
        self.norm = nn.LayerNorm(c_out, eps=eps, elementwise_affine=True, bias=False, dtype=dtype, device=device)

    def forward(self, x, mask):
        if mask is not None:
            x = x * mask[:, None, :, None].to(x.dtype)
        x = self.conv(x.to(self.conv.weight.dtype))
        x = torch.relu(self.norm(x.permute(0, 2, 3, 1)).permute(0, 3, 1, 2))
        return x, (mask[:, ::2] if mask is not None else None)


class _Subsample(nn.Module):
    def __init__(self, cfg: Gemma4AudioConfig, device=None):
        super().__init__()
        c0, c1 = cfg.subsampling_conv_channels
        self.layer0 = _SubsampleLayer(1, c0, cfg.norm_eps, cfg.dtype, device)
        self.layer1 = _SubsampleLayer(c0, c1, cfg.norm_eps, cfg.dtype, device)
        self.input_proj_linear = Linear((c0 // 4) * c1, cfg.hidden_size, False, cfg.dtype, device)

    def forward(self, feats, mask):
        x, mask = self.layer0(feats[:, None], mask)
        x, mask = self.layer1(x, mask)
        B, _, T, _ = x.shape
        return self.input_proj_linear(x.permute(0, 2, 3, 1).reshape(B, T, -1)), mask


class _FeedForward(nn.Module):
    def __init__(self, cfg: Gemma4AudioConfig, device=None):
        super().__init__()
        D = cfg.hidden_size
        self.cfg = cfg
        self.ffw_layer_1, self.ffw_layer_2 = ClippedLinear(cfg, D, 4 * D, device), ClippedLinear(cfg, 4 * D, D, device)
        self.pre_layer_norm = RMSNorm(D, 1e-6, False, cfg.dtype, device)
        self.post_layer_norm = RMSNorm(D, 1e-6, False, cfg.dtype, device)

    def forward(self, x):
        cfg = self.cfg
        h = self.pre_layer_norm(_clip(x, cfg.gradient_clipping))
        h = self.ffw_layer_2(TF.silu(self.ffw_layer_1(h)))
        return x + self.post_layer_norm(_clip(h, cfg.gradient_clipping)) * cfg.residual_weight


class _LightConv(nn.Module):
    def __init__(self, cfg: Gemma4AudioConfig, device=None):
        super().__init__()
        D = cfg.hidden_size
        self.cfg = cfg
        self.linear_start, self.linear_end = ClippedLinear(cfg, D, 2 * D, device), ClippedLinear(cfg, D, D, device)
        self.depthwise_conv1d = nn.Conv1d(D, D, cfg.conv_kernel_size, groups=D, bias=False, dtype=cfg.dtype, device=device)
        self.pre_layer_norm = RMSNorm(D, cfg.norm_eps, False, cfg.dtype, device)
        self.conv_norm = RMSNorm(D, cfg.norm_eps, False, cfg.dtype, device)

    def forward(self, x):
        h = TF.glu(self.linear_start(self.pre_layer_norm(x)), dim=-1)
        h = TF.pad(h.transpose(1, 2), (self.cfg.conv_kernel_size - 1, 0))            # causal: left padding only
        h = self.depthwise_conv1d(h).transpose(1, 2)
        h = TF.silu(self.conv_norm(_clip(h, self.cfg.gradient_clipping)))
        return x + self.linear_end(h)


class _LocalAttention(nn.Module):
    def __init__(self, cfg: Gemma4AudioConfig, device=None):
        super().__init__()
        D, N = cfg.hidden_size, cfg.num_heads
        self.cfg, self.H = cfg, D // N
        self.q_proj, self.k_proj = ClippedLinear(cfg, D, D, device), ClippedLinear(cfg, D, D, device)
        self.v_proj, self.post = ClippedLinear(cfg, D, D, device), ClippedLinear(cfg, D, D, device)
        self.relative_k_proj = Linear(D, D, False, cfg.dtype, device)
        self.per_dim_scale = nn.Parameter(torch.zeros(self.H, dtype=cfg.dtype, device=device))
        self.q_scale = (self.H ** -0.5) / math.log(2)
        self.k_scale = math.log(1 + math.e) / math.log(2)

    def forward(self, x, rel_pos, allowed):
        """x [B, T, D]; rel_pos [P, D] sinusoids of the distances past .. -future; allowed [B, T, T] bool."""
        cfg = self.cfg
        B, T, _ = x.shape
        N, H = cfg.num_heads, self.H
        past, future = cfg.attention_context_left - 1, cfg.attention_context_right
        q = self.q_proj(x).float().view(B, T, N, H) * self.q_scale * TF.softplus(self.per_dim_scale.float())
        k = self.k_proj(x).float().view(B, T, N, H) * self.k_scale
        v = self.v_proj(x).float().view(B, T, N, H)
        r = self.relative_k_proj(rel_pos).float().view(-1, N, H)                       # [P, N, H], index = past - distance
        s = torch.einsum("btnh,bsnh->bnts", q, k)
        bd = torch.einsum("btnh,pnh->bntp", q, r)                                      # [B, N, T, P]
        dist = torch.arange(T, device=x.device)[:, None] - torch.arange(T, device=x.device)[None, :]   # t - s
        inside = (dist <= past) & (dist >= -future)
        idx = (past - dist).clamp(0, r.shape[0] - 1)
        s = s + torch.where(inside, bd.gather(-1, idx.expand(B, N, T, T)), torch.zeros((), device=x.device))
        s = cfg.attention_logit_cap * torch.tanh(s / cfg.attention_logit_cap)
        s = s.masked_fill(~allowed[:, None], cfg.attention_invalid_logits_value)
        o = torch.einsum("bnts,bsnh->btnh", torch.softmax(s, -1), v).reshape(B, T, N * H)
        return self.post(o.to(self.post.linear.weight.dtype))


class _Layer(nn.Module):
    def __init__(self, cfg: Gemma4AudioConfig, device=None):
        super().__init__()
        D = cfg.hidden_size
        self.cfg = cfg
        self.feed_forward1, self.feed_forward2 = _FeedForward(cfg, device), _FeedForward(cfg, device)
        self.self_attn, self.lconv1d = _LocalAttention(cfg, device), _LightConv(cfg, device)
        self.norm_pre_attn = RMSNorm(D, 1e-6, False, cfg.dtype, device)
        self.norm_post_attn = RMSNorm(D, 1e-6, False, cfg.dtype, device)
        self.norm_out = RMSNorm(D, 1e-6, False, cfg.dtype, device)

    def forward(self, x, rel_pos, allowed):
        g = self.cfg.gradient_clipping
        x = self.feed_forward1(x)
        a = self.self_attn(self.norm_pre_attn(_clip(x, g)), rel_pos, allowed)
        x = x + self.norm_post_attn(_clip(a, g))
        x = self.feed_forward2(self.lconv1d(x))
        return self.norm_out(_clip(x, g))


class Gemma4AudioTower(nn.Module):
    def __init__(self, cfg: Gemma4AudioConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.subsample_conv_projection = _Subsample(cfg, device)
        self.layers = nn.ModuleList([_Layer(cfg, device) for _ in range(cfg.num_layers)])
        self.output_proj = Linear(cfg.hidden_size, cfg.output_proj_dims, True, cfg.dtype, device)

    def _relative_positions(self, device, dtype):
        cfg = self.cfg
        n = cfg.hidden_size // 2
        inc = math.log(10000.0) / max(n - 1, 1)
        inv = torch.exp(torch.arange(n, device=device, dtype=torch.float32) * -inc)
        d = torch.arange(cfg.attention_context_left - 1, -cfg.attention_context_right - 1, -1, device=device,
                         dtype=torch.float32)[:, None]
        return torch.cat([torch.sin(d * inv), torch.cos(d * inv)], -1).to(dtype)

    def forward(self, input_features, input_features_mask=None):
        """input_features [B, T, mel]; mask [B, T] true = real frame. Returns (frames [B, T/4, out], valid [B, T/4])."""
        cfg = self.cfg
        x, valid = self.subsample_conv_projection(input_features, input_features_mask)
        B, T, _ = x.shape
        if valid is None:
            valid = torch.ones(B, T, dtype=torch.bool, device=x.device)
        valid = valid.bool()
        dist = torch.arange(T, device=x.device)[:, None] - torch.arange(T, device=x.device)[None, :]
        # a frame sees itself and the context_left - 2 frames before it, and fewer than context_right after it
        band = ((dist >= 0) & (dist < cfg.attention_context_left - 1)) | ((dist < 0) & (-dist < cfg.attention_context_right))
        allowed = band[None] & valid[:, None, :] & valid[:, :, None]
        rel = self._relative_positions(x.device, x.dtype)
        for layer in self.layers:
            x = layer(x, rel, allowed)
        return self.output_proj(x), valid
