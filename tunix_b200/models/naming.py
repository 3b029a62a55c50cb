"""Model naming: HF ids <-> config ids <-> families (tunix/models/naming.py:136-171)."""
from __future__ import annotations

import dataclasses
import re

from .config import PRESETS, ModelConfig, get_config

_FAMILY_PATTERNS = [
    (r"llama[-_]?3", "llama3"), (r"qwen[-_]?3", "qwen3"), (r"qwen[-_]?2", "qwen2"), (r"deepseek[-_]?r1[-_]?distill[-_]?qwen", "qwen2"),
    (r"gemma[-_]?4", "gemma4"), (r"gemma[-_]?3", "gemma3"), (r"gemma[-_]?2", "gemma2"), (r"gemma", "gemma"),
]


@dataclasses.dataclass(frozen=True)
class ModelNaming:
    model_id: str        # e.g. "meta-llama/Llama-3.1-8B"
    model_name: str      # e.g. "llama-3.1-8b"
    family: str          # e.g. "llama3"
    config_id: str       # e.g. "llama3p1_8b"


def get_model_name_from_model_id(model_id: str) -> str:
    return model_id.split("/")[-1].lower()


def get_model_family(model_name: str) -> str:
    n = model_name.lower()
    for pat, fam in _FAMILY_PATTERNS:
        if re.search(pat, n):
            return fam
    raise ValueError(f"cannot determine the model family of {model_name!r}")


def get_model_config_id(model_name: str) -> str:
    """`llama-3.1-8b` -> `llama3p1_8b`, `qwen3-30b-a3b` -> `qwen3_30b_a3b`, `gemma-2-9b-it` -> `gemma2_9b`."""
    n = model_name.lower()
    n = re.sub(r"[-_](it|instruct|base|chat)$", "", n)
    n = n.replace("meta-", "")
    n = re.sub(r"^(llama|qwen|gemma)[-_]?(\d+)(?:\.(\d+))?", lambda m: f"{m.group(1)}{m.group(2)}" + (f"p{m.group(3)}" if m.group(3) else ""), n)
    n = n.replace("-", "_").replace(".", "p")
    if n.startswith("gemma4"):
        get_config("gemma4_e2b")          # Gemma-4 presets register on first use
    if n in PRESETS:
        return n
    # tolerate size suffix variants ("8b" vs "8B") and missing minor versions
    cands = [k for k in PRESETS if k.replace("_", "") == n.replace("_", "")]
    if cands:
        return cands[0]
    raise ValueError(f"no preset for {model_name!r} (normalised to {n!r}); known: {sorted(PRESETS)}")


def resolve(model_id: str) -> ModelNaming:
    name = get_model_name_from_model_id(model_id)
    return ModelNaming(model_id, name, get_model_family(name), get_model_config_id(name))


def config_for(model_id: str) -> ModelConfig:
    return get_config(resolve(model_id).config_id)
