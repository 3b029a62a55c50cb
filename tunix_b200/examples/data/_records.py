"""Record sources for the example pipelines. There is no dataset hub behind this package: records come from local
files (`.jsonl`, `.json` holding a list, `.parquet`, or a directory of such files taken in name order), from the
`datasets` package when it is installed and its cache already holds the dataset, or from a Python sequence."""
from __future__ import annotations

import json
import os
from typing import Any, Sequence

import numpy as np


def normalize_value(v: Any) -> Any:
    """bytes / numpy scalars and one-element arrays -> Python values (dataset readers hand back either)."""
    if isinstance(v, np.ndarray):
        flat = v.reshape(-1).tolist()
        return normalize_value(flat[0]) if len(flat) == 1 else [normalize_value(x) for x in flat]
    if isinstance(v, (bytes, np.bytes_)):
        return bytes(v).decode("utf-8")
    if isinstance(v, np.generic):
        return v.item()
    return v


def normalize_record(rec: dict) -> dict:
    return {k: (normalize_record(v) if isinstance(v, dict) else normalize_value(v)) for k, v in rec.items()}


def _read_file(path: str) -> list:
    if path.endswith(".jsonl"):
        with open(path) as f:
            return [json.loads(line) for line in f if line.strip()]
    if path.endswith(".json"):
        with open(path) as f:
            data = json.load(f)
        if isinstance(data, dict):                      # {"train": [...]} or column-major {"question": [...], ...}
            cols = [v for v in data.values() if isinstance(v, list)]
            if cols and all(not isinstance(x, dict) for x in cols[0]):
                return [dict(zip(data, row)) for row in zip(*data.values())]
            return [r for v in data.values() if isinstance(v, list) for r in v]
        return list(data)
    if path.endswith(".parquet"):
        import pyarrow.parquet as pq
        return pq.read_table(path).to_pylist()
    raise ValueError(f"unsupported data file {path!r} (use .jsonl, .json or .parquet)")


def load_records(source, split: str = "train") -> list:
    """`source`: a sequence of dicts, a file, a directory (files named `<split>*` are preferred when present), or a
    hub name `repo[:config]` resolved through the `datasets` package from its local cache."""
    if not isinstance(source, (str, os.PathLike)):
        return [normalize_record(dict(r)) for r in source]
    path = os.fspath(source)
    if os.path.isdir(path):
        files = sorted(f for f in os.listdir(path) if f.endswith((".jsonl", ".json", ".parquet")))
        preferred = [f for f in files if f.startswith(split)]
        files = preferred or files
        if not files:
            raise FileNotFoundError(f"no .jsonl / .json / .parquet file under {path!r}")
        return [normalize_record(r) for f in files for r in _read_file(os.path.join(path, f))]
    if os.path.isfile(path):
        return [normalize_record(r) for r in _read_file(path)]
    try:
        import datasets
    except ImportError as e:
        raise FileNotFoundError(f"{path!r} is neither a file nor a directory, and the `datasets` package that could resolve "
                                "it as a hub name is not installed") from e
    name, _, config = path.partition(":")
    return [normalize_record(dict(r)) for r in datasets.load_dataset(name, config or None, split=split)]


def shuffled(records: Sequence, seed: int) -> list:
    idx = np.random.default_rng(seed).permutation(len(records))
    return [records[i] for i in idx]
