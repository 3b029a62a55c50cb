"""Model configuration and the preset zoo.

One `ModelConfig` describes every decoder family the framework trains: Llama 3.x,
Qwen2.5, Qwen3 (dense and MoE), Gemma 1/2/3 (text). Presets follow the reference's
preset tables (tunix/models/llama3/model.py:103-187, tunix/models/qwen2/model.py:118-236,
tunix/models/qwen3/model.py:188-354, tunix/models/gemma/model.py:112-214,
tunix/models/gemma3/model.py:129-316) with HF shapes where the two disagree
(Gemma-2 MLP width, Llama rope theta honoured instead of ignored).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch


@dataclass
class ShardingConfig:
    """Named mesh axes each tensor class is split over (tunix/models/llama3/model.py:47-82)."""

    emb_vd: tuple = ("tp", "fsdp")
    emb_dv: tuple = ("fsdp", "tp")
    q_weight_dnh: tuple = ("fsdp", "tp", None)
    kv_weight_dnh: tuple = ("fsdp", "tp", None)
    o_weight_nhd: tuple = ("tp", None, "fsdp")
    ffw_weight_df: tuple = ("fsdp", "tp")
    ffw_weight_fd: tuple = ("tp", "fsdp")
    rms_norm_weight: tuple = ("tp",)
    act_btd: tuple = ("fsdp", None, "tp")
    act_btf: tuple = ("fsdp", None, "tp")
    act_btnh: tuple = ("fsdp", None, "tp", None)
    exp_weight_edf: tuple = ("fsdp", None, "tp")
    score_weight_d1: tuple = ("fsdp", None)

    @staticmethod
    def get_default_sharding(is_sampling: bool = False) -> "ShardingConfig":
        if not is_sampling:
            return ShardingConfig()
        strip = lambda spec: tuple(None if a == "fsdp" else a for a in spec)  # noqa: E731
        cfg = ShardingConfig()
        for f in dataclasses.fields(cfg):
            if not f.name.startswith("act_"):
                setattr(cfg, f.name, strip(getattr(cfg, f.name)))
        cfg.act_btd = ("fsdp", None, None)
        return cfg


class RematConfig:
    NONE = "none"        # keep every activation
    BLOCK = "block"      # recompute attention / MLP blocks
    DECODER = "decoder"  # recompute whole decoder layers (keep layer inputs only)


@dataclass
class ModelConfig:
    family: str = "llama3"
    num_layers: int = 2
    vocab_size: int = 1024
    embed_dim: int = 256
    hidden_dim: int = 1024
    num_heads: int = 4
    head_dim: int = 64
    num_kv_heads: int = 2
    rope_theta: float = 10000.0
    local_rope_theta: Optional[float] = None      # Gemma-3 local layers
    rope_scale_factor: float = 1.0                # Gemma-3 global layers
    rope_llama3_scaling: Optional[dict] = None
    norm_eps: float = 1e-6
    weight_tying: bool = False
    qkv_bias: bool = False                        # Qwen2
    qk_norm: bool = False                         # Qwen3, Gemma-3
    norm_add_one: bool = False                    # Gemma: scale is (1 + w)
    embed_scale: bool = False                     # Gemma: embeddings * sqrt(D)
    activation: str = "silu"                      # "silu" (SwiGLU) or "gelu" (GeGLU)
    attn_logit_softcap: float = 0.0               # Gemma-2
    final_logit_softcap: float = 0.0              # Gemma-2
    sliding_window: int = 0
    layer_pattern: Sequence[str] = ("global",)    # repeated over layers: "global" / "local"
    post_norms: bool = False                      # Gemma-2/3 post-attention and post-ffw norms
    query_pre_attn_scalar: Optional[float] = None
    # MoE (Qwen3-MoE)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_hidden_dim: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    # numerics / memory
    dtype: torch.dtype = torch.float32
    remat_config: str = RematConfig.NONE
    use_flash_attention: bool = True
    max_position: int = 8192
    logprob_chunk: int = 2048
    shd_config: ShardingConfig = field(default_factory=ShardingConfig)

    def layer_type(self, i: int) -> str:
        return self.layer_pattern[i % len(self.layer_pattern)]

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def num_params(self) -> int:
        D, F, V = self.embed_dim, self.hidden_dim, self.vocab_size
        attn = D * self.num_heads * self.head_dim * 2 + D * self.num_kv_heads * self.head_dim * 2
        if self.is_moe:
            mlp = self.num_experts * 3 * D * self.moe_hidden_dim + D * self.num_experts
        else:
            mlp = 3 * D * F
        per_layer = attn + mlp + 2 * D
        head = 0 if self.weight_tying else V * D
        return self.num_layers * per_layer + V * D + head + D

    def replace(self, **kw) -> "ModelConfig":
        return dataclasses.replace(self, **kw)

    # ------------------------------------------------------------------ presets
    @classmethod
    def tiny_llama(cls) -> "ModelConfig":
        """2-layer Llama-style decoder used by the CPU correctness config."""
        return cls(family="llama3", num_layers=2, vocab_size=1024, embed_dim=256, hidden_dim=1024, num_heads=4,
                   head_dim=64, num_kv_heads=2, rope_theta=10000.0, norm_eps=1e-6)

    @classmethod
    def llama3p2_1b(cls):
        return cls(family="llama3", num_layers=16, vocab_size=128256, embed_dim=2048, hidden_dim=8192, num_heads=32,
                   head_dim=64, num_kv_heads=8, rope_theta=500000.0, norm_eps=1e-5, weight_tying=True)

    @classmethod
    def llama3p2_3b(cls):
        return cls(family="llama3", num_layers=28, vocab_size=128256, embed_dim=3072, hidden_dim=8192, num_heads=24,
                   head_dim=128, num_kv_heads=8, rope_theta=500000.0, norm_eps=1e-5, weight_tying=True)

    @classmethod
    def llama3p1_8b(cls):
        return cls(family="llama3", num_layers=32, vocab_size=128256, embed_dim=4096, hidden_dim=14336, num_heads=32,
                   head_dim=128, num_kv_heads=8, rope_theta=500000.0, norm_eps=1e-5)

    @classmethod
    def llama3p1_70b(cls):
        return cls(family="llama3", num_layers=80, vocab_size=128256, embed_dim=8192, hidden_dim=28672, num_heads=64,
                   head_dim=128, num_kv_heads=8, rope_theta=500000.0, norm_eps=1e-5)

    @classmethod
    def llama3p1_405b(cls):
        return cls(family="llama3", num_layers=126, vocab_size=128256, embed_dim=16384, hidden_dim=53248,
                   num_heads=128, head_dim=128, num_kv_heads=8, rope_theta=500000.0, norm_eps=1e-5)

    @classmethod
    def _qwen2(cls, L, D, F, N, K, tie):
        return cls(family="qwen2", num_layers=L, vocab_size=151936, embed_dim=D, hidden_dim=F, num_heads=N,
                   head_dim=D // N, num_kv_heads=K, rope_theta=1000000.0, norm_eps=1e-6, qkv_bias=True,
                   weight_tying=tie)

    @classmethod
    def qwen2p5_0p5b(cls):
        return cls._qwen2(24, 896, 4864, 14, 2, True)

    @classmethod
    def qwen2p5_1p5b(cls):
        return cls._qwen2(28, 1536, 8960, 12, 2, True)

    @classmethod
    def qwen2p5_3b(cls):
        return cls._qwen2(36, 2048, 11008, 16, 2, True)

    @classmethod
    def qwen2p5_7b(cls):
        cfg = cls._qwen2(28, 3584, 18944, 28, 4, False)
        cfg.vocab_size = 152064
        return cfg

    @classmethod
    def deepseek_r1_distill_qwen_1p5b(cls):
        return cls._qwen2(28, 1536, 8960, 12, 2, False)

    @classmethod
    def _qwen3(cls, L, D, F, N, K, tie=False, H=128):
        return cls(family="qwen3", num_layers=L, vocab_size=151936, embed_dim=D, hidden_dim=F, num_heads=N,
                   head_dim=H, num_kv_heads=K, rope_theta=1000000.0, norm_eps=1e-6, qk_norm=True, weight_tying=tie)

    @classmethod
    def qwen3_0p6b(cls):
        return cls._qwen3(28, 1024, 3072, 16, 8, True)

    @classmethod
    def qwen3_1p7b(cls):
        return cls._qwen3(28, 2048, 6144, 16, 8, True)

    @classmethod
    def qwen3_4b(cls):
        return cls._qwen3(36, 2560, 9728, 32, 8, True)

    @classmethod
    def qwen3_8b(cls):
        return cls._qwen3(36, 4096, 12288, 32, 8)

    @classmethod
    def qwen3_14b(cls):
        return cls._qwen3(40, 5120, 17408, 40, 8)

    @classmethod
    def qwen3_32b(cls):
        return cls._qwen3(64, 5120, 25600, 64, 8)

    @classmethod
    def qwen3_30b_a3b(cls):
        cfg = cls._qwen3(48, 2048, 6144, 32, 4)
        cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_hidden_dim = 128, 8, 768
        cfg.router_aux_loss_coef = 0.001
        return cfg

    @classmethod
    def _gemma(cls, **kw):
        base = dict(family="gemma", vocab_size=256000, norm_eps=1e-6, norm_add_one=True, embed_scale=True,
                    activation="gelu", weight_tying=True, rope_theta=10000.0)
        base.update(kw)
        return cls(**base)

    @classmethod
    def gemma_2b(cls):
        return cls._gemma(num_layers=18, embed_dim=2048, hidden_dim=16384, num_heads=8, head_dim=256, num_kv_heads=1)

    @classmethod
    def gemma_7b(cls):
        return cls._gemma(num_layers=28, embed_dim=3072, hidden_dim=24576, num_heads=16, head_dim=256,
                          num_kv_heads=16)

    @classmethod
    def gemma2_2b(cls):
        return cls._gemma(family="gemma2", num_layers=26, embed_dim=2304, hidden_dim=9216, num_heads=8, head_dim=256,
                          num_kv_heads=4, attn_logit_softcap=50.0, final_logit_softcap=30.0, sliding_window=4096,
                          layer_pattern=("local", "global"), post_norms=True, query_pre_attn_scalar=256.0)

    @classmethod
    def gemma2_9b(cls):
        return cls._gemma(family="gemma2", num_layers=42, embed_dim=3584, hidden_dim=14336, num_heads=16,
                          head_dim=256, num_kv_heads=8, attn_logit_softcap=50.0, final_logit_softcap=30.0,
                          sliding_window=4096, layer_pattern=("local", "global"), post_norms=True,
                          query_pre_attn_scalar=256.0)

    @classmethod
    def _gemma3(cls, L, D, F, N, K, H=256, window=1024, vocab=262144, qpas=None):
        return cls._gemma(family="gemma3", vocab_size=vocab, num_layers=L, embed_dim=D, hidden_dim=F, num_heads=N,
                          head_dim=H, num_kv_heads=K, sliding_window=window,
                          layer_pattern=("local",) * 5 + ("global",), post_norms=True, qk_norm=True,
                          rope_theta=1000000.0, local_rope_theta=10000.0, query_pre_attn_scalar=qpas or float(H))

    @classmethod
    def gemma3_270m(cls):
        return cls._gemma3(18, 640, 2048, 4, 1, window=512)

    @classmethod
    def gemma3_1b(cls):
        return cls._gemma3(26, 1152, 6912, 4, 1, window=512)

    @classmethod
    def gemma3_4b(cls):
        cfg = cls._gemma3(34, 2560, 10240, 8, 4)
        cfg.rope_scale_factor = 8.0
        return cfg

    @classmethod
    def gemma3_12b(cls):
        cfg = cls._gemma3(48, 3840, 15360, 16, 8)
        cfg.rope_scale_factor = 8.0
        return cfg

    @classmethod
    def gemma3_27b(cls):
        cfg = cls._gemma3(62, 5376, 21504, 32, 16, H=128, qpas=168.0)
        cfg.rope_scale_factor = 8.0
        return cfg


PRESETS = {name: getattr(ModelConfig, name) for name in dir(ModelConfig)
           if not name.startswith("_") and name not in ("replace", "layer_type", "num_params", "is_moe")
           and isinstance(ModelConfig.__dict__.get(name), classmethod)}


def get_config(name: str) -> ModelConfig:
    """Look up a preset by config id (e.g. `llama3p1_8b`, `qwen3_8b`, `gemma2_9b`)."""
    key = name.lower().replace("-", "_").replace(".", "p")
    if key.startswith("gemma4") and key not in PRESETS:
        from .gemma4 import Gemma4Config          # registered on first use: gemma4 imports this module
        for n in ("gemma4_e2b", "gemma4_e4b", "gemma4_12b", "gemma4_31b", "gemma4_26b_a4b"):
            PRESETS[n] = getattr(Gemma4Config, n)
            PRESETS[n + "_it"] = getattr(Gemma4Config, n)
    if key not in PRESETS:
        raise KeyError(f"unknown model config '{name}'; known: {sorted(PRESETS)}")
    return PRESETS[key]()
