"""Load HF safetensors checkpoints into the in-framework decoder (tunix/models/safetensors_loader.py:73-541).

Weights keep the HF `[out, in]` layout, so loading is: memory-map each file, map the HF key to the module
path with a per-family regex table, optionally stack per-expert tensors (Qwen3-MoE), cast, and copy straight
into the (possibly sharded) destination parameter. One tensor is resident on the host at a time.
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Callable, Optional

import torch

# (HF key regex, our parameter name template). Applied in order; first match wins.
_COMMON = [
    (r"model\.embed_tokens\.weight", "embed_tokens"),
    (r"model\.norm\.weight", "norm.weight"),
    (r"lm_head\.weight", "lm_head"),
    (r"model\.layers\.(\d+)\.self_attn\.(q|k|v|o)_proj\.(weight|bias)", r"layers.\1.self_attn.\2_proj.\3"),
    (r"model\.layers\.(\d+)\.self_attn\.(q|k)_norm\.weight", r"layers.\1.self_attn.\2_norm.weight"),
    (r"model\.layers\.(\d+)\.mlp\.(gate|up|down)_proj\.weight", r"layers.\1.mlp.\2_proj.weight"),
    (r"model\.layers\.(\d+)\.input_layernorm\.weight", r"layers.\1.input_layernorm.weight"),
]
_KEY_MAPS = {
    "default": _COMMON + [
        (r"model\.layers\.(\d+)\.post_attention_layernorm\.weight", r"layers.\1.post_attention_layernorm.weight"),
        (r"model\.layers\.(\d+)\.mlp\.gate\.weight", r"layers.\1.mlp.router.weight"),
        (r"model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight", r"layers.\1.mlp.\3_proj#\2"),
    ],
    # Gemma-2/3 use four norms per layer; HF's `post_attention_layernorm` is the norm applied to the
    # attention OUTPUT, and `pre_feedforward_layernorm` is the MLP input norm.
    "gemma_post_norms": _COMMON + [
        (r"model\.layers\.(\d+)\.post_attention_layernorm\.weight", r"layers.\1.post_attn_norm.weight"),
        (r"model\.layers\.(\d+)\.pre_feedforward_layernorm\.weight", r"layers.\1.post_attention_layernorm.weight"),
        (r"model\.layers\.(\d+)\.post_feedforward_layernorm\.weight", r"layers.\1.post_ffw_norm.weight"),
    ],
    # Gemma-4 keeps the HF norm names; "a|b" = the tensor is split in equal parts along its second-to-last axis
    "gemma4": _COMMON + [
        (r"model\.embed_tokens_per_layer\.weight", "embed_tokens_per_layer"),
        (r"model\.per_layer_(model_projection|projection_norm)\.weight", r"per_layer_\1.weight"),
        (r"model\.layers\.(\d+)\.(post_attention|pre_feedforward|post_feedforward)_layernorm\.weight", r"layers.\1.\2_layernorm.weight"),
        (r"model\.layers\.(\d+)\.(post_feedforward_layernorm_1|post_feedforward_layernorm_2|pre_feedforward_layernorm_2)\.weight",
         r"layers.\1.\2.weight"),
        (r"model\.layers\.(\d+)\.(per_layer_input_gate|per_layer_projection|post_per_layer_input_norm)\.weight", r"layers.\1.\2.weight"),
        (r"model\.layers\.(\d+)\.layer_scalar", r"layers.\1.layer_scalar"),
        (r"model\.layers\.(\d+)\.router\.proj\.weight", r"layers.\1.moe.router.weight"),
        (r"model\.layers\.(\d+)\.router\.scale", r"layers.\1.moe.router_scale"),
        (r"model\.layers\.(\d+)\.router\.per_expert_scale", r"layers.\1.moe.per_expert_scale"),
        (r"model\.layers\.(\d+)\.experts\.gate_up_proj", r"layers.\1.moe.gate_proj|layers.\1.moe.up_proj"),
        (r"model\.layers\.(\d+)\.experts\.down_proj", r"layers.\1.moe.down_proj"),
    ],
}


def key_map_for(cfg) -> list:
    if cfg.family == "gemma4":
        return _KEY_MAPS["gemma4"]
    return _KEY_MAPS["gemma_post_norms" if cfg.post_norms else "default"]


def map_key(hf_key: str, table: list) -> Optional[str]:
    hf_key = re.sub(r"^language_model\.", "", hf_key)                 # language_model.model.layers... (Gemma 3)
    hf_key = re.sub(r"^model\.language_model\.", "model.", hf_key)    # model.language_model.layers... (Gemma 4)
    for pat, repl in table:
        m = re.fullmatch(pat, hf_key)
        if m:
            return m.expand(repl)
    return None


def inverse_map_key(our_key: str, cfg) -> str:
    """Our parameter name -> HF key (used by the saver)."""
    if our_key == "embed_tokens":
        return "model.embed_tokens.weight"
    if our_key == "lm_head":
        return "lm_head.weight"
    if our_key == "norm.weight":
        return "model.norm.weight"
    k = "model." + our_key
    if cfg.post_norms:
        k = k.replace(".post_attention_layernorm.", ".pre_feedforward_layernorm.")
        k = k.replace(".post_attn_norm.", ".post_attention_layernorm.")
        k = k.replace(".post_ffw_norm.", ".post_feedforward_layernorm.")
    k = k.replace(".mlp.router.weight", ".mlp.gate.weight")
    return k


def load_safetensors_into(model, path: str, dtype: Optional[torch.dtype] = None, strict: bool = True,
                          preprocess_fn: Optional[Callable] = None) -> list:
    """Load every `*.safetensors` under `path` (a file or a directory) into `model`. Returns unused HF keys."""
    from safetensors import safe_open
    files = [path] if os.path.isfile(path) else sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {path}")
    table = key_map_for(model.config)
    params = dict(model.named_parameters())
    params.update({n: b for n, b in model.named_buffers() if n.endswith("layer_scalar")})
    seen, unused = set(), []
    with torch.no_grad():
        for f in files:
            with safe_open(f, framework="pt", device="cpu") as sf:
                for key in sf.keys():
                    name = map_key(key, table)
                    if name is None:
                        unused.append(key)
                        continue
                    t = sf.get_tensor(key)
                    if preprocess_fn is not None:
                        t = preprocess_fn(name, t)
                    if "|" in name:
                        names = name.split("|")
                        for nm, part in zip(names, t.chunk(len(names), dim=-2)):
                            params[nm].copy_(part.to(params[nm].device, dtype or params[nm].dtype))
                            seen.add((nm, None))
                        continue
                    expert = None
                    if "#" in name:
                        name, e = name.split("#")
                        expert = int(e)
                    if name not in params:
                        if name == "lm_head" and model.config.weight_tying:
                            continue
                        unused.append(key)
                        continue
                    dst = params[name]
                    dst = dst[expert] if expert is not None else dst
                    if dst.shape != t.shape:
                        raise ValueError(f"shape mismatch for {key} -> {name}: checkpoint {tuple(t.shape)} vs model {tuple(dst.shape)}")
                    dst.copy_(t.to(dst.device, dtype or dst.dtype))
                    seen.add((name, expert))
    if strict:
        missing = []
        for n, p in params.items():
            if "lora_" in n or (n, None) in seen:
                continue
            if p.dim() == 3 and n.endswith(("gate_proj", "up_proj", "down_proj")) and model.config.is_moe:
                missing += [f"{n}#{e}" for e in range(p.shape[0]) if (n, e) not in seen]
            elif (n, None) not in seen:
                missing.append(n)
        if missing:
            raise KeyError(f"parameters missing from checkpoint: {missing[:8]}{'...' if len(missing) > 8 else ''}")
    return unused


def create_model_from_safe_tensors(path: str, config, device=None, dtype: Optional[torch.dtype] = None):
    """Build the model of `config` and fill it from the checkpoint at `path`."""
    from .transformer import create_model
    if dtype is not None:
        config = config.replace(dtype=dtype)
    model = create_model(config, device=device, init=False)
    load_safetensors_into(model, path)
    return model
