"""Dataset loading for the DeepScaleR agentic GRPO recipe (tunix/cli/recipes/deepscaler_data.py:27-76).

The training set is a JSON file of {"problem", "answer", ...} records, the evaluation set (AIME) a parquet file with the
same fields. Every element becomes {"prompts", "question", "answer"} with the step-by-step / boxed-answer instruction
appended to the question. Files are read from local paths (pandas; parquet through pyarrow)."""
from __future__ import annotations

import json
import random
from typing import Optional

INSTRUCTION = "Let's think step by step, and put your final answer within \\boxed{}."


def _to_prompt(item: dict) -> dict:
    question = item.get("question", item.get("problem", ""))
    answer = item.get("answer", item.get("ground_truth", ""))
    return {"prompts": f"{question} {INSTRUCTION}", "question": question, "answer": answer}


def _read_records(path: str) -> list:
    if path.endswith(".parquet"):
        import pandas as pd
        return pd.read_parquet(path).to_dict("records")
    with open(path) as f:
        text = f.read().strip()
    if text.startswith("["):
        return json.loads(text)
    return [json.loads(line) for line in text.splitlines() if line.strip()]      # JSON lines


def create_dataset(train_data_path: str, eval_data_path: Optional[str] = None, shuffle: bool = False, seed: int = 42):
    """-> (train rows, eval rows or None); rows are dicts with "prompts", "question", "answer"."""
    train = [_to_prompt(r) for r in _read_records(train_data_path)]
    if shuffle:
        random.Random(seed).shuffle(train)
    evals = [_to_prompt(r) for r in _read_records(eval_data_path)] if eval_data_path else None
    return train, evals
