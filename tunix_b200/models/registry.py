"""Model family registry (role of tunix/models/registry.py): one table from family name to how a model of that
family is configured, loaded and named, so new families plug in without touching AutoModel."""
from __future__ import annotations

import dataclasses
from typing import Callable, Optional

from . import config as config_lib


@dataclasses.dataclass(frozen=True)
class FamilyEntry:
    family: str
    config_fn: Callable[[str], "config_lib.ModelConfig"]      # preset name -> config
    hf_prefixes: tuple                                          # Hugging Face id prefixes of this family
    chat_template: str                                          # parser name in rl.agentic.parser
    notes: str = ""


_FAMILIES: dict = {}


def register_family(entry: FamilyEntry) -> None:
    _FAMILIES[entry.family] = entry


def get_family(name: str) -> FamilyEntry:
    if name not in _FAMILIES:
        raise KeyError(f"unknown model family {name!r}; known: {sorted(_FAMILIES)}")
    return _FAMILIES[name]


def family_of_hf_id(model_id: str) -> Optional[FamilyEntry]:
    low = model_id.lower().split("/")[-1]
    best = None
    for e in _FAMILIES.values():
        for p in e.hf_prefixes:
            if low.startswith(p) and (best is None or len(p) > best[0]):
                best = (len(p), e)
    return best[1] if best else None


def families() -> list:
    return sorted(_FAMILIES)


for _fam, _pref, _tmpl in (("llama3", ("llama-3", "meta-llama-3", "llama3"), "llama"),
                           ("qwen2", ("qwen2", "deepseek-r1-distill-qwen"), "qwen"),
                           ("qwen3", ("qwen3",), "qwen"),
                           ("gemma", ("gemma-2b", "gemma-7b", "gemma-1.1"), "gemma"),
                           ("gemma2", ("gemma-2-",), "gemma"),
                           ("gemma3", ("gemma-3-",), "gemma"),
                           ("gemma4", ("gemma-4-",), "gemma4")):
    register_family(FamilyEntry(_fam, config_lib.get_config, _pref, _tmpl))
