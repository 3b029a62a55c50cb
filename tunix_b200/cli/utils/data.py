"""Datasets for the CLI (tunix/cli/utils/data.py, tunix/examples/data/*): tokenise -> pad -> `TrainingInput`.

Sources: `synthetic` (uniform token ids, for benchmarks), `jsonl` (records with `text`, or `src`/`dst` for
translation-style SFT, or `question`/`answer` for RL prompts), `module` (a Python module exposing
`create_datasets(...)`)."""
from __future__ import annotations

import importlib
import json
import os
from typing import Iterator

import numpy as np

from ...sft.peft_trainer import TrainingInput


def _pad_batch(rows, masks, length, pad_id):
    ids = np.full((len(rows), length), pad_id, np.int64)
    m = np.zeros((len(rows), length), np.float32)
    for i, (r, mk) in enumerate(zip(rows, masks)):
        r, mk = r[:length], mk[:length]
        ids[i, :len(r)], m[i, :len(r)] = r, mk
    return TrainingInput(ids, m)


def synthetic_sft(batch_size, seq_len, vocab_size, num_batches, seed=0, prompt_len=0) -> Iterator[TrainingInput]:
    rng = np.random.default_rng(seed)
    for _ in range(num_batches):
        ids = rng.integers(0, vocab_size, (batch_size, seq_len), dtype=np.int64)
        mask = np.ones((batch_size, seq_len), np.float32)
        mask[:, :prompt_len] = 0
        yield TrainingInput(ids, mask)


def chat_row_tokens(messages, tokenizer, chat_parser):
    """Token ids of a conversation and a loss mask that is 1 on the assistant's turns only (their end marker
    included, the role header the template puts before them excluded)."""
    ids = list(tokenizer.encode(chat_parser.bos())) if chat_parser.bos() else []
    mask = [0.0] * len(ids)
    header = tokenizer.encode(chat_parser.generation_prompt) if chat_parser.generation_prompt else []
    for m in messages:
        t = tokenizer.encode(chat_parser.render_message(m))
        learn = m.get("role") == "assistant"
        skip = len(header) if learn and t[:len(header)] == header else 0
        ids += t
        mask += [0.0] * skip + [1.0 if learn else 0.0] * (len(t) - skip)
    return ids, mask


def jsonl_sft(path, tokenizer, batch_size, max_target_length, epochs=1, chat_parser=None) -> Iterator[TrainingInput]:
    """Rows are {"text"}, {"src", "dst"} or {"messages": [{"role", "content"}, ...]} (chat rows, e.g. the
    trajectory explorer's `export-sft`; the loss covers the assistant's turns)."""
    recs = [json.loads(l) for l in open(path) if l.strip()]
    pad = tokenizer.pad_id()
    if chat_parser is None and any("messages" in r for r in recs):
        from ...rl.agentic.parser.chat_template_parser import get_parser
        chat_parser = get_parser("qwen", tokenizer)
    for _ in range(epochs):
        for s0 in range(0, len(recs) - batch_size + 1, batch_size):
            rows, masks = [], []
            for r in recs[s0:s0 + batch_size]:
                if "messages" in r:
                    t, m = chat_row_tokens(r["messages"], tokenizer, chat_parser)
                    rows.append(t[:max_target_length])
                    masks.append(m[:max_target_length])
                elif "src" in r:
                    p = tokenizer.encode(r["src"])
                    c = tokenizer.encode(r["dst"]) + [tokenizer.eos_id()]
                    rows.append(([tokenizer.bos_id()] if tokenizer.bos_id() is not None else []) + p + c)
                    masks.append([0.0] * (len(rows[-1]) - len(c)) + [1.0] * len(c))
                else:
                    t = tokenizer.encode(r["text"]) + [tokenizer.eos_id()]
                    rows.append(t)
                    masks.append([1.0] * len(t))
            yield _pad_batch(rows, masks, max_target_length, pad)


def jsonl_prompts(path, batch_size, apply_template=None, epochs=1) -> Iterator[dict]:
    recs = [json.loads(l) for l in open(path) if l.strip()]
    for _ in range(epochs):
        for s0 in range(0, len(recs) - batch_size + 1, batch_size):
            chunk = recs[s0:s0 + batch_size]
            prompts = [r.get("question", r.get("prompt", "")) for r in chunk]
            if apply_template:
                prompts = [apply_template(p) for p in prompts]
            yield {"prompts": prompts, "answer": [r.get("answer") for r in chunk]}


def synthetic_prompts(batch_size, prompt_len, vocab_size, num_batches, seed=2) -> Iterator[dict]:
    rng = np.random.default_rng(seed)
    for _ in range(num_batches):
        yield {"prompt_token_ids": rng.integers(3, vocab_size, (batch_size, prompt_len)).tolist()}


def create_datasets(hp, tokenizer, vocab_size):
    c = hp.config
    n = c["num_batches"] or (c["training_config"]["max_steps"] or 10) * (c["training_config"].get("gradient_accumulation_steps") or 1)
    if c["data_source"] == "synthetic":
        return (synthetic_sft(c["batch_size"], c["max_target_length"], vocab_size, n),
                synthetic_sft(c["batch_size"], c["max_target_length"], vocab_size, min(c["num_test_batches"], 2), seed=99))
    if c["data_source"] == "jsonl":
        tr = os.path.join(c["data_directory"], c["dataset_name"] or "train.jsonl")
        ev = os.path.join(c["data_directory"], "eval.jsonl")
        return (jsonl_sft(tr, tokenizer, c["batch_size"], c["max_target_length"], c["num_train_epochs"]),
                jsonl_sft(ev, tokenizer, c["batch_size"], c["max_target_length"]) if os.path.exists(ev) else None)
    if c["data_source"] == "module":
        mod = importlib.import_module(c["data_module"])
        return mod.create_datasets(c, tokenizer)
    raise ValueError(f"unknown data_source {c['data_source']!r}")
