"""Grade-school math prompts for RL recipes (tunix/examples/data/math_dataset.py:30-222): question → prompt in the
reasoning / answer tag format, gold answer from the text after `####`."""
from __future__ import annotations

import logging
from typing import Optional

from ...utils import token_sanitization
from . import _records

log = logging.getLogger(__name__)
reasoning_start, reasoning_end = "<reasoning>", "</reasoning>"
solution_start, solution_end = "<answer>", "</answer>"

SYSTEM_PROMPT = (f"You are given a problem. Think about the problem and provide your reasoning. Place it between "
                 f"{reasoning_start} and {reasoning_end}. Then, provide the final answer (i.e., just one numerical value) "
                 f"between {solution_start} and {solution_end}.")
TEMPLATE = "<start_of_turn>user\n{system_prompt}\n\n{question}<end_of_turn>\n<start_of_turn>model"


def extract_hash_answer(text: str) -> Optional[str]:
    if "####" not in text:
        return None
    return text.split("####")[1].strip().replace(",", "")


def apply_template(records, tokenizer=None, tokenize: bool = False, add_generation_prompt: bool = True) -> list:
    """`{"prompts", "question", "answer"}` per record. With a tokenizer that has a chat template the system prompt and
    the question go through it; otherwise the fixed Gemma-style template is used. Control tokens inside the question
    text are neutralised first, so that dataset text cannot open or close a turn."""
    if tokenizer is not None and hasattr(tokenizer, "apply_chat_template"):
        fmt = lambda q: tokenizer.apply_chat_template([{"role": "system", "content": SYSTEM_PROMPT}, {"role": "user", "content": q}],
                                                      tokenize=tokenize, add_generation_prompt=add_generation_prompt)
    else:
        fmt = lambda q: TEMPLATE.format(system_prompt=SYSTEM_PROMPT, question=q)
    out = []
    for rec in records:
        rec = _records.normalize_record(dict(rec))
        q = token_sanitization.sanitize_control_tokens(rec["question"])
        out.append({"prompts": fmt(q), "question": q, "answer": extract_hash_answer(str(rec["answer"]))})
    return out


def _parse_huggingface_dataset_name(dataset_name: str):
    """`repo:config` → (repo, config); `org/repo` → (repo, "default"); a bare name → (name, None)."""
    if ":" in dataset_name:
        name, config = dataset_name.split(":", maxsplit=1)
        return name, config or None
    if "/" in dataset_name:
        return dataset_name, "default"
    return dataset_name, None


def create_dataset(data_source: str, dataset, tokenizer=None, split: str = "train", apply_chat_template_to_dataset: bool = False,
                   shuffle_seed: Optional[int] = 42) -> list:
    """`data_source`: "local" (a .parquet / .jsonl / .json file or a directory of them) or "huggingface" (a hub name
    resolved from the local cache of the `datasets` package). Returns the (shuffled) records, templated on request."""
    if data_source == "local":
        recs = _records.load_records(dataset, split)
    elif data_source == "huggingface":
        name, config = _parse_huggingface_dataset_name(str(dataset))
        recs = _records.load_records(f"{name}:{config}" if config else name, split)
    else:
        raise ValueError(f"Unsupported combination of dataset='{dataset}' and data_source='{data_source}'")
    if shuffle_seed is not None:
        recs = _records.shuffled(recs, shuffle_seed)
    return apply_template(recs, tokenizer) if apply_chat_template_to_dataset else recs
