"""Export to HF safetensors with LoRA merged as `W + (B @ A) * alpha / r`
(tunix/models/safetensors_saver.py:30-126); tokenizer / config files of the source directory are copied."""
from __future__ import annotations

import os
import shutil
from typing import Optional

import torch

from ..lora import merged_weight
from .safetensors_loader import inverse_map_key
from .transformer import Linear


def _gemma4_export(model, tensors: dict) -> dict:
    """Gemma-4 key names of a causal-LM checkpoint: the layer scalars are buffers, the expert gate and up weights
    are stored as one tensor, router tensors live under `router.`."""
    out = {}
    for name, t in tensors.items():
        if name == "embed_tokens":
            out["model.embed_tokens.weight"] = t
        elif name == "embed_tokens_per_layer":
            out["model.embed_tokens_per_layer.weight"] = t
        elif name == "lm_head":
            out["lm_head.weight"] = t
        elif name.endswith(".moe.up_proj"):
            continue
        elif name.endswith(".moe.gate_proj"):
            base = name[: -len(".moe.gate_proj")]
            out[f"model.{base}.experts.gate_up_proj"] = torch.cat([t, tensors[base + ".moe.up_proj"]], dim=1).contiguous()
        elif name.endswith(".moe.down_proj"):
            out["model." + name.replace(".moe.down_proj", ".experts.down_proj")] = t
        elif ".moe.router" in name or ".moe.per_expert_scale" in name:
            k = name.replace(".moe.router.weight", ".router.proj.weight").replace(".moe.router_scale", ".router.scale")
            out["model." + k.replace(".moe.per_expert_scale", ".router.per_expert_scale")] = t
        else:
            out["model." + name] = t
    for name, b in model.named_buffers():
        if name.endswith("layer_scalar"):
            out["model." + name] = b.detach().contiguous().cpu()
    return out


def state_dict_for_export(model, merge_lora: bool = True) -> dict:
    cfg = model.config
    out = {}
    lin = {n: m for n, m in model.named_modules() if isinstance(m, Linear)}
    for name, p in model.named_parameters():
        if "lora_" in name or name.startswith("_distill_"):
            continue
        mod_name = name.rsplit(".", 1)[0] if "." in name else ""
        if name.endswith(".weight") and mod_name in lin and merge_lora and lin[mod_name].lora_a is not None:
            t = merged_weight(lin[mod_name])
        elif name.endswith(".weight") and mod_name in lin and lin[mod_name].quant is not None:
            t = lin[mod_name].base_weight()
        else:
            t = p.detach()
        if cfg.family == "gemma4":
            out[name] = t.contiguous().cpu()
            continue
        if cfg.is_moe and p.dim() == 3 and name.endswith(("gate_proj", "up_proj", "down_proj")):
            base = inverse_map_key(name, cfg).rsplit(".", 1)
            for e in range(p.shape[0]):
                out[f"{base[0]}.experts.{e}.{base[1]}.weight"] = t[e].contiguous().cpu()
            continue
        out[inverse_map_key(name, cfg)] = t.contiguous().cpu()
    if cfg.family == "gemma4":
        return _gemma4_export(model, out)
    return out


def save_lora_merged_model_as_safetensors(model, output_dir: str, source_dir: Optional[str] = None,
                                          merge_lora: bool = True) -> str:
    from safetensors.torch import save_file
    os.makedirs(output_dir, exist_ok=True)
    path = os.path.join(output_dir, "model.safetensors")
    save_file(state_dict_for_export(model, merge_lora), path, metadata={"format": "pt"})
    if source_dir:
        for f in os.listdir(source_dir):
            if f.endswith((".json", ".model", ".txt", ".tiktoken")) and not f.endswith(".safetensors.index.json"):
                shutil.copy2(os.path.join(source_dir, f), os.path.join(output_dir, f))
    return path
