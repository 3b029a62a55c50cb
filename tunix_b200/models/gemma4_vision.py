"""Gemma 4 vision encoder and the multimodal front end (tunix/models/gemma4/vision.py, model.py).

Images arrive already cut into patches by the host processor (`processors/image_processor.py`): `pixel_values`
`[B, P, 3 * patch^2]` in [0, 1] and `pixel_position_ids` `[B, P, 2]` = (x, y) of each patch, (-1, -1) for padding,
so images of different aspect ratios share a batch.

  patches -> 2 * (x - 0.5) -> linear -> + learned x-table[x] + y-table[y]
          -> encoder layers (four RMSNorms, bidirectional attention among the valid patches, GeGLU MLP, optional
             clipping of every linear layer's input and output); rotary embedding in two dimensions: the first
             half of each head rotates with the patch's x, the second half with its y
          -> average over k x k patch cells, scaled by sqrt(width) (-> P / k^2 soft tokens, with a validity mask)
          -> optional standardisation -> RMSNorm without scale -> projection into the decoder's width

Attention runs on the tcgen05 flash kernel (`causal=False`, valid / padding patches as two segments) when the
tower is bf16 on CUDA.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from ..ops import functional as F
from .transformer import Linear, RMSNorm


@dataclass
class Gemma4VisionConfig:
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_layers: int = 16
    num_heads: int = 12
    num_kv_heads: int = 12
    head_dim: int = 64
    norm_eps: float = 1e-6
    rope_theta: float = 100.0
    pooling_kernel_size: int = 3
    patch_size: int = 16
    position_embedding_size: int = 10 * 1024
    use_clipped_linears: bool = False
    standardize: bool = False
    image_token_id: int = 258880
    dtype: torch.dtype = torch.bfloat16


class ClippedLinear(nn.Module):
    """Linear layer whose input and output are clamped to stored ranges (the small checkpoints were trained so)."""

    def __init__(self, cfg: Gemma4VisionConfig, n_in: int, n_out: int, device=None):
        super().__init__()
        self.linear = Linear(n_in, n_out, False, cfg.dtype, device)
        self.clip = cfg.use_clipped_linears
        if self.clip:
            for name, v in (("input_min", -math.inf), ("input_max", math.inf), ("output_min", -math.inf), ("output_max", math.inf)):
                self.register_buffer(name, torch.tensor(v, device=device))

    def forward(self, x):
        if self.clip:
            x = torch.clamp(x, self.input_min.to(x.dtype), self.input_max.to(x.dtype))
        y = self.linear(x)
        if self.clip:
            y = torch.clamp(y, self.output_min.to(y.dtype), self.output_max.to(y.dtype))
        return y


def rope_2d(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x [B, P, heads, H]; pos [B, P, 2]. The first H/2 channels rotate (half-split pairs) with pos[..., 0], the
    second H/2 with pos[..., 1]; each half uses the frequencies theta^(-2i / (H/2))."""
    H = x.shape[-1]
    part = 2 * (H // 4)
    inv = 1.0 / (theta ** (torch.arange(0, part, 2, device=x.device, dtype=torch.float32) / part))
    out = []
    xf = x.float()
    for d in range(2):
        ang = pos[..., d].float()[..., None] * inv                     # [B, P, part/2]
        c, s = ang.cos()[:, :, None, :], ang.sin()[:, :, None, :]
        a, b = xf[..., d * part: d * part + part // 2], xf[..., d * part + part // 2: (d + 1) * part]
        out += [a * c - b * s, b * c + a * s]
    if 2 * part < H:
        out.append(xf[..., 2 * part:])
    return torch.cat(out, -1).to(x.dtype)


class VisionAttention(nn.Module):
    def __init__(self, cfg: Gemma4VisionConfig, device=None):
        super().__init__()
        self.cfg = cfg
        D, N, K, H = cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        self.q_proj, self.k_proj = ClippedLinear(cfg, D, N * H, device), ClippedLinear(cfg, D, K * H, device)
        self.v_proj, self.o_proj = ClippedLinear(cfg, D, K * H, device), ClippedLinear(cfg, N * H, D, device)
        self.q_norm = RMSNorm(H, cfg.norm_eps, False, cfg.dtype, device)
        self.k_norm = RMSNorm(H, cfg.norm_eps, False, cfg.dtype, device)
        self.register_buffer("_unit", torch.ones(H, dtype=cfg.dtype, device=device), persistent=False)

    def forward(self, x, pos, seg):
        cfg = self.cfg
        B, P, _ = x.shape
        N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        q = rope_2d(self.q_norm(self.q_proj(x).view(B, P, N, H)), pos, cfg.rope_theta)
        k = rope_2d(self.k_norm(self.k_proj(x).view(B, P, K, H)), pos, cfg.rope_theta)
        v = F.rmsnorm(self.v_proj(x).view(B, P, K, H), self._unit, cfg.norm_eps, False)
        o = F.attention(q, k, v, scale=1.0, causal=False, seg_q=seg, seg_k=seg)
        return self.o_proj(o.reshape(B, P, N * H))


class VisionMLP(nn.Module):
    def __init__(self, cfg: Gemma4VisionConfig, device=None):
        super().__init__()
        self.gate_proj = ClippedLinear(cfg, cfg.hidden_size, cfg.intermediate_size, device)
        self.up_proj = ClippedLinear(cfg, cfg.hidden_size, cfg.intermediate_size, device)
        self.down_proj = ClippedLinear(cfg, cfg.intermediate_size, cfg.hidden_size, device)

    def forward(self, x):
        return self.down_proj(F.glu(self.gate_proj(x), self.up_proj(x), "gelu"))


class VisionLayer(nn.Module):
    def __init__(self, cfg: Gemma4VisionConfig, device=None):
        super().__init__()
        mk = lambda: RMSNorm(cfg.hidden_size, cfg.norm_eps, False, cfg.dtype, device)  # noqa: E731
        self.self_attn, self.mlp = VisionAttention(cfg, device), VisionMLP(cfg, device)
        self.input_layernorm, self.post_attention_layernorm = mk(), mk()
        self.pre_feedforward_layernorm, self.post_feedforward_layernorm = mk(), mk()

    def forward(self, x, pos, seg):
        x = x + self.post_attention_layernorm(self.self_attn(self.input_layernorm(x), pos, seg))
        return x + self.post_feedforward_layernorm(self.mlp(self.pre_feedforward_layernorm(x)))


class _Embedder(nn.Module):
    def __init__(self, cfg: Gemma4VisionConfig, device=None):
        super().__init__()
        self.input_proj = Linear(3 * cfg.patch_size ** 2, cfg.hidden_size, False, cfg.dtype, device)
        self.position_embedding_table = nn.Parameter(torch.ones(2, cfg.position_embedding_size, cfg.hidden_size,
                                                                dtype=cfg.dtype, device=device))

    def forward(self, pixels, pos, pad):
        x = self.input_proj((2.0 * (pixels.float() - 0.5)).to(self.input_proj.weight.dtype))
        p = pos.clamp(min=0)
        pe = self.position_embedding_table[0][p[..., 0]] + self.position_embedding_table[1][p[..., 1]]
        return x + torch.where(pad[..., None], torch.zeros_like(pe), pe)


class _Encoder(nn.Module):
    def __init__(self, cfg: Gemma4VisionConfig, device=None):
        super().__init__()
        self.layers = nn.ModuleList([VisionLayer(cfg, device) for _ in range(cfg.num_layers)])


class Gemma4VisionTower(nn.Module):
    """Module names follow the Hugging Face checkpoint (`patch_embedder`, `encoder.layers.N...`, `std_bias`), so a
    checkpoint's vision state dict loads as is."""

    def __init__(self, cfg: Gemma4VisionConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.patch_embedder = _Embedder(cfg, device)
        self.encoder = _Encoder(cfg, device)
        if cfg.standardize:
            self.register_buffer("std_bias", torch.zeros(cfg.hidden_size, dtype=cfg.dtype, device=device))
            self.register_buffer("std_scale", torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device))

    def forward(self, pixel_values, pixel_position_ids):
        """Returns (soft tokens [B, P / k^2, width], valid [B, P / k^2])."""
        cfg = self.cfg
        pos = pixel_position_ids.long()
        pad = (pos == -1).all(-1)
        x = self.patch_embedder(pixel_values, pos, pad)
        seg = (~pad).to(torch.int32)
        for layer in self.encoder.layers:
            x = layer(x, pos, seg)
        x = x.masked_fill(pad[..., None], 0.0)
        B, P, D = x.shape
        k = cfg.pooling_kernel_size
        out_len = P // (k * k)
        valid = ~pad
        if out_len != P:
            p = pos.clamp(min=0)
            max_x = p[..., 0].max(-1, keepdim=True)[0] + 1
            cell = torch.div(p, k, rounding_mode="floor")
            cell = cell[..., 0] + (max_x // k) * cell[..., 1]                              # [B, P]
            w = torch.nn.functional.one_hot(cell, out_len).float() / (k * k)              # [B, P, out]
            x = (w.transpose(1, 2) @ x.float()).to(x.dtype)
            valid = ~(w == 0).all(1)
        x = x * math.sqrt(D)
        if cfg.standardize:
            x = (x - self.std_bias) * self.std_scale
        return x, valid


class Gemma4MultimodalEmbedder(nn.Module):
    """Soft tokens -> decoder width: RMSNorm without a scale, then a projection."""

    def __init__(self, width: int, embed_dim: int, eps: float, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.embedding_projection = Linear(width, embed_dim, False, dtype, device)
        self.eps = eps
        self.register_buffer("_unit", torch.ones(width, dtype=dtype, device=device), persistent=False)

    def forward(self, soft):
        return self.embedding_projection(F.rmsnorm(soft, self._unit, self.eps, False))


def splice_soft_tokens(emb: torch.Tensor, is_slot: torch.Tensor, soft: torch.Tensor, valid: torch.Tensor) -> torch.Tensor:
    """emb [B, T, D]; is_slot [B, T] true at placeholder tokens; soft [B, S, D] with validity [B, S]. The k-th
    placeholder of a row receives the k-th valid soft token of that row."""
    B, T, D = emb.shape
    order = torch.argsort((~valid).to(torch.int8), dim=1, stable=True)                  # valid ones first, in order
    rank = (torch.cumsum(is_slot.long(), 1) - 1).clamp(min=0, max=soft.shape[1] - 1)
    picked = soft.gather(1, order.gather(1, rank)[..., None].expand(B, T, D))
    return torch.where(is_slot[..., None], picked.to(emb.dtype), emb)


class Gemma4Multimodal(nn.Module):
    """Gemma 4 decoder with the vision (and optionally the audio) encoder in front.
    `forward(tokens, pixel_values=..., pixel_position_ids=..., input_features=..., input_features_mask=...)` puts
    the k-th valid soft token of a row over its k-th placeholder token of that modality; per-layer inputs of those
    positions come from the padding token, as in the reference. With `bidirectional_images` the tokens of one
    image attend to each other in both directions (the 31B / 26B-A4B checkpoints)."""

    def __init__(self, language_model, vision_config: Gemma4VisionConfig, bidirectional_images: bool = False,
                 pad_token_id: int = 0, audio_config=None, device=None):
        super().__init__()
        self.language_model = language_model
        self.vision_config = vision_config
        self.audio_config = audio_config
        self.vision_tower = Gemma4VisionTower(vision_config, device)
        lm_cfg = language_model.config
        self.embed_vision = Gemma4MultimodalEmbedder(vision_config.hidden_size, lm_cfg.embed_dim, vision_config.norm_eps,
                                                     lm_cfg.dtype, device)
        if audio_config is not None:
            from .gemma4_audio import Gemma4AudioTower
            self.audio_tower = Gemma4AudioTower(audio_config, device)
            self.embed_audio = Gemma4MultimodalEmbedder(audio_config.output_proj_dims, lm_cfg.embed_dim, audio_config.norm_eps,
                                                        lm_cfg.dtype, device)
        self.bidirectional_images = bidirectional_images
        self.pad_token_id = pad_token_id
        self.config = lm_cfg

    @torch.no_grad()
    def init_encoder_weights(self, seed: int = 0, std: float = 0.02) -> "Gemma4Multimodal":
        """Random normal(0, std) matrices for the encoders and their embedders (the decoder has its own
        `init_weights`); norm scales and position tables keep their constructor values."""
        mods = [self.vision_tower, self.embed_vision] + ([self.audio_tower, self.embed_audio] if self.audio_config is not None else [])
        dev = next(self.vision_tower.parameters()).device
        gen = torch.Generator(device=dev).manual_seed(seed)
        for m in mods:
            for name, p in m.named_parameters():
                if p.dim() >= 2 and "position_embedding_table" not in name:
                    p.normal_(0.0, std, generator=gen)
                elif name.endswith("bias"):
                    p.zero_()
        return self

    def encode_images(self, pixel_values, pixel_position_ids):
        soft, valid = self.vision_tower(pixel_values, pixel_position_ids)
        return self.embed_vision(soft), valid

    def encode_audio(self, input_features, input_features_mask=None):
        frames, valid = self.audio_tower(input_features, input_features_mask)
        return self.embed_audio(frames), valid

    # what the dense `Sampler` asks of its model besides `forward`
    def init_cache(self, *a, **kw):
        return self.language_model.init_cache(*a, **kw)

    def compute_final_logits(self, hidden):
        return self.language_model.compute_final_logits(hidden)

    def forward(self, input_tokens, pixel_values=None, pixel_position_ids=None, input_features=None,
                input_features_mask=None, positions=None, segment_ids=None, skip_lm_head: bool = False, cache=None, **kw):
        lm, vc, ac = self.language_model, self.vision_config, self.audio_config
        if pixel_values is None and input_features is None:
            return lm(input_tokens, positions=positions, segment_ids=segment_ids, skip_lm_head=skip_lm_head, cache=cache, **kw)
        cfg = lm.config
        B, T = input_tokens.shape
        is_img = input_tokens == vc.image_token_id
        is_aud = (input_tokens == ac.audio_token_id) if ac is not None else torch.zeros_like(is_img)
        safe = torch.where(is_img | is_aud, torch.full_like(input_tokens, self.pad_token_id), input_tokens)
        emb = F.embedding(safe, lm.embed_tokens, math.sqrt(cfg.embed_dim) if cfg.embed_scale else 1.0)
        if pixel_values is not None:
            soft, valid = self.encode_images(pixel_values, pixel_position_ids)
            emb = splice_soft_tokens(emb, is_img, soft.reshape(B, -1, soft.shape[-1]), valid.reshape(B, -1))
        if input_features is not None:
            soft, valid = self.encode_audio(input_features, input_features_mask)
            emb = splice_soft_tokens(emb, is_aud, soft.reshape(B, -1, soft.shape[-1]), valid.reshape(B, -1))
        ple = lm.per_layer_inputs(safe, emb) if cfg.per_layer_input_dim else None
        mask = None
        if self.bidirectional_images and pixel_values is not None:
            from . import cache_utils
            start = is_img & ~torch.nn.functional.pad(is_img, (1, 0))[:, :-1]
            spans = torch.where(is_img, torch.cumsum(start.long(), 1), torch.zeros_like(input_tokens, dtype=torch.long))
            pos = torch.arange(T, device=input_tokens.device)
            mask = torch.stack([cache_utils.prefill_mask(pos, pos, bidirectional_span=spans[b]) for b in range(B)])
        return lm.forward_embeddings(emb, positions=positions, cache=cache, attention_mask=mask, segment_ids=segment_ids,
                                     skip_lm_head=skip_lm_head, per_layer_inputs=ple)

    def token_logprobs(self, *a, **kw):
        return self.language_model.token_logprobs(*a, **kw)
