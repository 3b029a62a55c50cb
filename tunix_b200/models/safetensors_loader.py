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
}


def key_map_for(cfg) -> list:
    return _KEY_MAPS["gemma_post_norms" if cfg.post_norms else "default"]


def map_key(hf_key: str, table: list) -> Optional[str]:
    hf_key = re.sub(r"^language_model\.", "", hf_key)
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
            if "lora_" in n:
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
    from .transformer import Transformer
    if dtype is not None:
        config = config.replace(dtype=dtype)
    model = Transformer(config, device=device)
    load_safetensors_into(model, path)
    return model
