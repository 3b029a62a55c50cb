"""`ModelConfig` from a Hugging Face `config.json`, so that a checkpoint directory is self-describing and needs no
preset name (the reference maps model ids to hand-written presets, tunix/models/naming.py and automodel.py; a
directory whose sizes differ from every preset has no entry there).

Covers the decoder families of `models/transformer.py`: Llama 3.x, Qwen2 / 2.5, Qwen3 (dense and MoE), Gemma 1 / 2 /
3 text. Multimodal wrappers (`text_config` inside) are unwrapped to their text decoder."""
from __future__ import annotations

import json
import os
from typing import Optional, Union

import torch

from .config import ModelConfig

_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def _rope_theta(c: dict, default: float) -> float:
    rp = c.get("rope_parameters")
    if isinstance(rp, dict):
        if "rope_theta" in rp:
            return float(rp["rope_theta"])
        for v in rp.values():                               # per layer type (Gemma 3): the global one
            if isinstance(v, dict) and "rope_theta" in v:
                return float(rp.get("full_attention", v).get("rope_theta", v["rope_theta"]))
    return float(c.get("rope_theta", default))


def _layer_pattern(c: dict, default: tuple) -> tuple:
    lt = c.get("layer_types")
    if lt:
        names = tuple("local" if "sliding" in t else "global" for t in lt)
        for period in range(1, len(names) + 1):             # shortest repeating unit
            if all(names[i] == names[i % period] for i in range(len(names))):
                return names[:period]
    return default


def config_from_hf(src: Union[str, dict], dtype: Optional[torch.dtype] = None, **overrides) -> ModelConfig:
    """`src`: a checkpoint directory, a `config.json` path or the parsed dict."""
    if isinstance(src, str):
        path = os.path.join(src, "config.json") if os.path.isdir(src) else src
        with open(path, encoding="utf-8") as f:
            c = json.load(f)
    else:
        c = dict(src)
    outer = c
    if isinstance(c.get("text_config"), dict):
        c = dict(c["text_config"])
    mt = c.get("model_type", outer.get("model_type", ""))
    D, N = int(c["hidden_size"]), int(c["num_attention_heads"])
    if dtype is None:
        dtype = _DTYPES.get(str(c.get("torch_dtype") or c.get("dtype") or outer.get("torch_dtype") or outer.get("dtype") or "bfloat16")
                            .replace("torch.", ""), torch.bfloat16)
    kw = dict(num_layers=int(c["num_hidden_layers"]), vocab_size=int(c["vocab_size"]), embed_dim=D,
              hidden_dim=int(c.get("intermediate_size", 4 * D)), num_heads=N, head_dim=int(c.get("head_dim") or D // N),
              num_kv_heads=int(c.get("num_key_value_heads") or N), norm_eps=float(c.get("rms_norm_eps", 1e-6)),
              weight_tying=bool(c.get("tie_word_embeddings", outer.get("tie_word_embeddings", False))),
              max_position=int(c.get("max_position_embeddings", 8192)), dtype=dtype)
    if mt == "llama":
        kw.update(family="llama3", rope_theta=_rope_theta(c, 500000.0))
        rs = c.get("rope_scaling") or (c.get("rope_parameters") if isinstance(c.get("rope_parameters"), dict) else None)
        if isinstance(rs, dict) and (rs.get("rope_type") or rs.get("type")) == "llama3":
            kw["rope_llama3_scaling"] = {k: rs[k] for k in ("factor", "low_freq_factor", "high_freq_factor",
                                                            "original_max_position_embeddings") if k in rs}
    elif mt == "qwen2":
        kw.update(family="qwen2", rope_theta=_rope_theta(c, 1000000.0), qkv_bias=True)
    elif mt in ("qwen3", "qwen3_moe"):
        kw.update(family="qwen3", rope_theta=_rope_theta(c, 1000000.0), qk_norm=True)
        if mt == "qwen3_moe":
            kw.update(num_experts=int(c["num_experts"]), num_experts_per_tok=int(c["num_experts_per_tok"]),
                      moe_hidden_dim=int(c["moe_intermediate_size"]), norm_topk_prob=bool(c.get("norm_topk_prob", True)),
                      router_aux_loss_coef=float(c.get("router_aux_loss_coef", 0.0)))
    elif mt in ("gemma", "gemma2", "gemma3_text", "gemma3"):
        kw.update(family={"gemma3_text": "gemma3"}.get(mt, mt), norm_add_one=True, embed_scale=True, activation="gelu",
                  weight_tying=bool(c.get("tie_word_embeddings", True)), rope_theta=_rope_theta(c, 10000.0))
        if mt != "gemma":
            kw.update(post_norms=True, sliding_window=int(c.get("sliding_window") or 0),
                      query_pre_attn_scalar=float(c.get("query_pre_attn_scalar", kw["head_dim"])))
        if mt == "gemma2":
            kw.update(attn_logit_softcap=float(c.get("attn_logit_softcapping") or 0.0),
                      final_logit_softcap=float(c.get("final_logit_softcapping") or 0.0),
                      layer_pattern=_layer_pattern(c, ("local", "global")))
        if mt in ("gemma3_text", "gemma3"):
            n = int(c.get("sliding_window_pattern") or 6)
            rp = c.get("rope_parameters") if isinstance(c.get("rope_parameters"), dict) else {}
            local = (rp.get("sliding_attention") or {}).get("rope_theta", c.get("rope_local_base_freq", 10000.0))
            glob = rp.get("full_attention") or {}
            scaling = c.get("rope_scaling") or {}
            kw.update(qk_norm=True, layer_pattern=_layer_pattern(c, ("local",) * (n - 1) + ("global",)),
                      local_rope_theta=float(local), rope_theta=float(glob.get("rope_theta", c.get("rope_theta", 1000000.0))),
                      rope_scale_factor=float(glob.get("factor", scaling.get("factor", 1.0)) or 1.0),
                      final_logit_softcap=float(c.get("final_logit_softcapping") or 0.0))
    else:
        raise ValueError(f"no decoder in this framework for Hugging Face model_type {mt!r}")
    kw.update(overrides)
    return ModelConfig(**kw)
