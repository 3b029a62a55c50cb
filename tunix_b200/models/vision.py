"""SigLIP-style vision tower and the multimodal front end of Gemma-3
(tunix/models/gemma3/vision.py:80-682, merge_embeddings.py:21-57, model.py:330-370,1080-1145).

    image [H, W, 3] -> 14x14 patches -> linear patch embedding + learned position embedding
      -> `depth` pre-LayerNorm encoder blocks (bidirectional multi-head attention, GELU MLP) -> final LayerNorm
      -> average pool the 64x64 patch grid down to 16x16 = 256 soft tokens per image
      -> RMSNorm + linear projection into the language model's embedding space
      -> written over the embeddings of the image placeholder tokens of the prompt.

Attention runs on the framework's flash-attention kernel with `causal=False` when the tower is bf16 on CUDA
(head dim 72 falls back to the PyTorch path: the kernel covers head dims 64 / 128 / 256). Image tokens of one
image attend to each other in both directions inside the language model; `image_span_ids` produces the ids that
`models.cache_utils.prefill_mask(bidirectional_span=...)` turns into the mask.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF


@dataclasses.dataclass
class VisionConfig:
    image_height: int = 896
    image_width: int = 896
    image_channels: int = 3
    patch_size: tuple = (14, 14)
    width: int = 1152
    depth: int = 27
    mlp_dim: Optional[int] = 4304
    num_heads: int = 16
    num_mm_tokens_per_image: int = 256
    image_mean: tuple = (127.5, 127.5, 127.5)
    image_std: tuple = (127.5, 127.5, 127.5)
    image_token_id: int = 262144          # placeholder id of one soft token in the prompt
    dtype: torch.dtype = torch.bfloat16

    @property
    def grid(self) -> tuple:
        return (self.image_height // self.patch_size[0], self.image_width // self.patch_size[1])

    @classmethod
    def siglip_so400m(cls, **kw) -> "VisionConfig":
        return cls(**kw)

    @classmethod
    def tiny(cls, **kw) -> "VisionConfig":
        base = dict(image_height=32, image_width=32, patch_size=(8, 8), width=64, depth=2, mlp_dim=128, num_heads=1,
                    num_mm_tokens_per_image=4, dtype=torch.float32)
        base.update(kw)
        return cls(**base)


class VisionAttention(nn.Module):
    def __init__(self, width: int, num_heads: int, dtype, device=None):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, width // num_heads
        mk = lambda: nn.Linear(width, width, bias=True, dtype=dtype, device=device)   # noqa: E731
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = mk(), mk(), mk(), mk()

    def forward(self, x):
        B, L, W = x.shape
        q, k, v = (p(x).view(B, L, self.num_heads, self.head_dim) for p in (self.q_proj, self.k_proj, self.v_proj))
        if x.is_cuda and x.dtype == torch.bfloat16 and self.head_dim in (64, 128, 256):
            from ..ops import functional as F
            o = F.attention(q, k, v, scale=1.0 / math.sqrt(self.head_dim), causal=False)
        else:
            o = TF.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
        return self.out_proj(o.reshape(B, L, W))


class EncoderBlock(nn.Module):
    def __init__(self, cfg: VisionConfig, device=None):
        super().__init__()
        W, dt = cfg.width, cfg.dtype
        self.norm1 = nn.LayerNorm(W, eps=1e-6, dtype=dt, device=device)
        self.attn = VisionAttention(W, cfg.num_heads, dt, device)
        self.norm2 = nn.LayerNorm(W, eps=1e-6, dtype=dt, device=device)
        hidden = cfg.mlp_dim or 4 * W
        self.fc1 = nn.Linear(W, hidden, dtype=dt, device=device)
        self.fc2 = nn.Linear(hidden, W, dtype=dt, device=device)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.fc2(TF.gelu(self.fc1(self.norm2(x)), approximate="tanh"))


class VisionTower(nn.Module):
    """images [B, N, H, W, C] (already normalised, see processors.ImageProcessor) -> soft tokens [B, N, P, width]."""

    def __init__(self, cfg: VisionConfig, device=None):
        super().__init__()
        self.cfg = cfg
        ph, pw = cfg.patch_size
        self.patch_embed = nn.Linear(ph * pw * cfg.image_channels, cfg.width, dtype=cfg.dtype, device=device)
        gh, gw = cfg.grid
        self.pos_embedding = nn.Parameter(torch.randn(1, gh * gw, cfg.width, dtype=cfg.dtype, device=device) / math.sqrt(cfg.width))
        self.blocks = nn.ModuleList([EncoderBlock(cfg, device) for _ in range(cfg.depth)])
        self.norm = nn.LayerNorm(cfg.width, eps=1e-6, dtype=cfg.dtype, device=device)

    def patchify(self, images: torch.Tensor) -> torch.Tensor:
        B, H, W, C = images.shape
        ph, pw = self.cfg.patch_size
        x = images.view(B, H // ph, ph, W // pw, pw, C).permute(0, 1, 3, 2, 4, 5)
        return x.reshape(B, (H // ph) * (W // pw), ph * pw * C)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, N = images.shape[:2]
        x = self.patchify(images.reshape(B * N, *images.shape[2:]).to(cfg.dtype))
        x = self.patch_embed(x) + self.pos_embedding
        for blk in self.blocks:
            x = blk(x)
        x = self.norm(x)
        gh, gw = cfg.grid
        side = int(math.isqrt(cfg.num_mm_tokens_per_image))
        if side * side != cfg.num_mm_tokens_per_image or gh % side or gw % side:
            raise ValueError("soft tokens per image must be a square that divides the patch grid")
        x = x.view(B * N, gh, gw, cfg.width).permute(0, 3, 1, 2)
        x = TF.avg_pool2d(x.float(), kernel_size=(gh // side, gw // side)).to(cfg.dtype)      # the "vision exit"
        return x.permute(0, 2, 3, 1).reshape(B, N, side * side, cfg.width)


class MultimodalProjector(nn.Module):
    """RMSNorm + projection of soft tokens into the language model's embedding space (model.py:330-370)."""

    def __init__(self, vision_width: int, embed_dim: int, eps: float = 1e-6, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.norm_weight = nn.Parameter(torch.zeros(vision_width, dtype=dtype, device=device))     # (1 + w) convention
        self.proj = nn.Parameter(torch.empty(vision_width, embed_dim, dtype=dtype, device=device))
        nn.init.normal_(self.proj, std=0.02)
        self.eps = eps

    def forward(self, soft: torch.Tensor) -> torch.Tensor:
        x = soft.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * (1.0 + self.norm_weight.float())
        return (x.to(self.proj.dtype) @ self.proj)


def merge_embeddings(text_embeddings: torch.Tensor, vision_embeddings: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """text [B, L, D]; vision [B, N, P, D]; mask [B, L] true at image placeholder tokens. The k-th true position
    of a row receives the k-th soft token of that row (images in order); rows with fewer placeholders than soft
    tokens use the leading ones, rows without placeholders are returned unchanged."""
    B, L, D = text_embeddings.shape
    flat = vision_embeddings.reshape(B, -1, D)
    rank = torch.cumsum(mask.long(), dim=1) - 1
    rank = rank.clamp(min=0, max=flat.shape[1] - 1)
    picked = flat.gather(1, rank[..., None].expand(B, L, D))
    return torch.where(mask[..., None].bool(), picked.to(text_embeddings.dtype), text_embeddings)


def image_span_ids(tokens: torch.Tensor, image_token_id: int, tokens_per_image: int) -> torch.Tensor:
    """[B, L] ints: 0 for text, k >= 1 for the tokens of the k-th image of the row (bidirectional spans)."""
    is_img = tokens == image_token_id
    idx = torch.cumsum(is_img.long(), 1) - 1
    return torch.where(is_img, idx // tokens_per_image + 1, torch.zeros_like(idx))


class Gemma3Multimodal(nn.Module):
    """A language model with a vision tower in front: `forward(tokens, images=...)` embeds, splices the projected
    soft tokens over the placeholders and runs the decoder with image spans attending bidirectionally."""

    def __init__(self, language_model, vision_config: VisionConfig, device=None):
        super().__init__()
        self.language_model = language_model
        self.vision_config = vision_config
        self.vision_tower = VisionTower(vision_config, device)
        lm_cfg = language_model.config
        self.projector = MultimodalProjector(vision_config.width, lm_cfg.embed_dim, lm_cfg.norm_eps, lm_cfg.dtype, device)
        self.config = lm_cfg

    def encode_images(self, images: torch.Tensor) -> torch.Tensor:
        if images.dim() == 4:
            images = images[:, None]
        return self.projector(self.vision_tower(images))

    def forward(self, input_tokens, images=None, positions=None, segment_ids=None, skip_lm_head: bool = False, **kw):
        lm, vc = self.language_model, self.vision_config
        if images is None:
            return lm(input_tokens, positions=positions, segment_ids=segment_ids, skip_lm_head=skip_lm_head, **kw)
        from ..models import cache_utils
        from ..ops import functional as F
        cfg = lm.config
        safe = torch.where(input_tokens == vc.image_token_id, torch.zeros_like(input_tokens), input_tokens)
        emb = F.embedding(safe, lm.embed_tokens, math.sqrt(cfg.embed_dim) if cfg.embed_scale else 1.0)
        emb = merge_embeddings(emb, self.encode_images(images), input_tokens == vc.image_token_id)
        B, T = input_tokens.shape
        spans = image_span_ids(input_tokens, vc.image_token_id, vc.num_mm_tokens_per_image)
        pos = torch.arange(T, device=input_tokens.device)
        mask = torch.stack([cache_utils.prefill_mask(pos, pos, bidirectional_span=spans[b]) for b in range(B)])
        return lm.forward_embeddings(emb, positions=positions, attention_mask=mask, skip_lm_head=skip_lm_head)

    def token_logprobs(self, *a, **kw):
        return self.language_model.token_logprobs(*a, **kw)
