"""Trajectory logging to CSV / JSONL / JSON with an asynchronous writer.

Serialisation goes through the native `_trajjson` module (csrc/pyext/trajjson.cc) when it is built:
`dumps_json` / `format_ndarray` release the GIL while formatting, so logging 10^5-element arrays does not
stall the training thread. The pure-Python versions below define the behaviour and are the fallback.

Mirrors tunix/utils/trajectory_logger.py (serialisation helpers :41-62, `AsyncTrajectoryLogger` :786-975):
a bounded queue feeds worker threads; `log(item)` never blocks the trainer longer than the queue allows;
`stop()` drains with a timeout; dataclasses, dicts, lists, numpy arrays/scalars are accepted.
"""
from __future__ import annotations

import csv
import dataclasses
import json
import math
import os
import queue
import threading
import time
from typing import Any, Literal, Optional

import numpy as np

try:  # native fast path
    if os.environ.get("TUNIX_B200_TRAJJSON_LIB"):           # another build of the module (the sanitizer build of the tests)
        import importlib.machinery
        import importlib.util
        _loader = importlib.machinery.ExtensionFileLoader(__package__ + "._trajjson", os.environ["TUNIX_B200_TRAJJSON_LIB"])
        _trajjson = importlib.util.module_from_spec(importlib.util.spec_from_loader(_loader.name, _loader))
        _loader.exec_module(_trajjson)
    else:
        from . import _trajjson  # type: ignore
except Exception:  # pragma: no cover - exercised only without the built module
    _trajjson = None

TrajectoryFileFormat = Literal["csv", "jsonl", "json"]


class SerializedArray(str):
    """A pre-formatted array: `repr()` is the unquoted bracketed text and `dumps_json` emits it verbatim."""

    def __repr__(self) -> str:
        return str(self)


if _trajjson is not None:
    _trajjson._set_serialized_array_type(SerializedArray)


def _py_scalar(v):
    if isinstance(v, (np.bool_,)):
        return bool(v)
    if isinstance(v, np.integer):
        return int(v)
    if isinstance(v, np.floating):
        return float(v)
    return v


def format_ndarray_py(arr: np.ndarray) -> str:
    return repr(np.asarray(arr).tolist())


def format_ndarray(arr: np.ndarray) -> SerializedArray:
    """Text identical to `repr(arr.tolist())`."""
    arr = np.asarray(arr)
    if _trajjson is not None and arr.dtype.kind in "iufb" and arr.dtype.itemsize in (1, 2, 4, 8) \
            and arr.dtype != np.float16:
        try:
            return SerializedArray(_trajjson.format_ndarray(arr))
        except TypeError:
            pass
    return SerializedArray(format_ndarray_py(arr))


def _to_jsonable(o: Any) -> Any:
    if isinstance(o, SerializedArray):
        return json.loads(str(o).replace("nan", "NaN").replace("inf", "Infinity").replace("True", "true").replace("False", "false"))
    if dataclasses.is_dataclass(o) and not isinstance(o, type):
        return _to_jsonable(dataclasses.asdict(o))
    if isinstance(o, dict):
        return {(k if isinstance(k, str) else ("true" if k is True else "false" if k is False else
                                               "null" if k is None else str(k))): _to_jsonable(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [_to_jsonable(v) for v in o]
    if isinstance(o, np.ndarray):
        return o.tolist()
    if isinstance(o, np.generic):
        return _py_scalar(o)
    if hasattr(o, "detach") and hasattr(o, "cpu"):  # torch tensor
        return o.detach().float().cpu().numpy().tolist() if o.dtype.is_floating_point else o.detach().cpu().numpy().tolist()
    if isinstance(o, (str, int, float, bool)) or o is None:
        return o
    return str(o)


def dumps_json_py(obj: Any, indent: int = -1) -> str:
    return json.dumps(_to_jsonable(obj), indent=None if indent < 0 else indent)


def dumps_json(obj: Any, indent: int = -1) -> str:
    """`json.dumps`-compatible text (ensure_ascii, NaN / Infinity tokens). ndarrays stay on one line."""
    if _trajjson is not None:
        try:
            return _trajjson.dumps_json(_strip_tensors(obj), indent)
        except (TypeError, ValueError, RecursionError):
            pass
    return dumps_json_py(obj, indent)


def _strip_tensors(o: Any) -> Any:
    """torch tensors -> numpy (bf16/fp16 widened); everything else untouched (shallow walk of containers)."""
    if hasattr(o, "detach") and hasattr(o, "cpu"):
        t = o.detach().cpu()
        if t.dtype.is_floating_point and t.element_size() < 4:
            t = t.float()
        return t.numpy()
    if isinstance(o, np.ndarray) and (o.dtype == np.float16 or o.dtype.kind not in "iufb"):
        return o.tolist()
    if isinstance(o, dict):
        return {k: _strip_tensors(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [_strip_tensors(v) for v in o]
    if dataclasses.is_dataclass(o) and not isinstance(o, type):
        return {f.name: _strip_tensors(getattr(o, f.name)) for f in dataclasses.fields(o)}
    return o


def _row_of(item: Any) -> dict:
    if dataclasses.is_dataclass(item) and not isinstance(item, type):
        item = {f.name: getattr(item, f.name) for f in dataclasses.fields(item)}
    if not isinstance(item, dict):
        item = {"value": item}
    return item


def log_item(log_path: str, item: Any, file_format: TrajectoryFileFormat = "jsonl") -> None:
    """Synchronously append one item."""
    os.makedirs(os.path.dirname(log_path) or ".", exist_ok=True)
    if file_format == "jsonl":
        with open(log_path, "a") as f:
            f.write(dumps_json(_row_of(item)) + "\n")
    elif file_format == "json":
        data = []
        if os.path.exists(log_path):
            with open(log_path) as f:
                data = json.load(f)
        data.append(json.loads(dumps_json(_row_of(item))))
        with open(log_path, "w") as f:
            json.dump(data, f)
    elif file_format == "csv":
        row = {k: (format_ndarray(v) if isinstance(v, np.ndarray) else
                   (dumps_json(v) if isinstance(v, (dict, list, tuple)) else v)) for k, v in _row_of(item).items()}
        exists = os.path.exists(log_path)
        with open(log_path, "a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(row))
            if not exists:
                w.writeheader()
            w.writerow(row)
    else:
        raise ValueError(f"unknown trajectory file format {file_format!r}")


class AsyncTrajectoryLogger:
    """Background writer: `log()` enqueues, worker threads serialise and append."""

    def __init__(self, log_dir: str, file_format: TrajectoryFileFormat = "jsonl", file_name: str = "trajectories",
                 max_queue_size: int = 1000, num_workers: int = 1, stop_timeout_sec: float = 15.0):
        self.log_path = os.path.join(log_dir, f"{file_name}.{file_format}")
        self.file_format = file_format
        self._q: queue.Queue = queue.Queue(maxsize=max_queue_size)
        self._lock = threading.Lock()
        self._stop_timeout = stop_timeout_sec
        self._errors: list = []
        self._dropped = 0
        self._workers = [threading.Thread(target=self._run, daemon=True, name=f"traj-log-{i}")
                         for i in range(max(1, num_workers))]
        self._stopped = False
        for w in self._workers:
            w.start()

    def _run(self):
        while True:
            item = self._q.get()
            try:
                if item is None:
                    return
                with self._lock:  # appends to one file are serialised; formatting releases the GIL
                    log_item(self.log_path, item, self.file_format)
            except Exception as e:  # keep logging alive; surface on stop()
                self._errors.append(e)
            finally:
                self._q.task_done()

    def log(self, item: Any, block: bool = True, timeout: Optional[float] = None) -> bool:
        if self._stopped:
            raise RuntimeError("logger already stopped")
        try:
            self._q.put(item, block=block, timeout=timeout)
            return True
        except queue.Full:
            self._dropped += 1
            return False

    @property
    def dropped(self) -> int:
        return self._dropped

    def flush(self, timeout: Optional[float] = None) -> bool:
        deadline = time.time() + (timeout if timeout is not None else self._stop_timeout)
        while self._q.unfinished_tasks and time.time() < deadline:
            time.sleep(0.005)
        return self._q.unfinished_tasks == 0

    def stop(self) -> None:
        if self._stopped:
            return
        self._stopped = True
        for _ in self._workers:
            self._q.put(None)
        for w in self._workers:
            w.join(self._stop_timeout)
        if self._errors:
            raise RuntimeError(f"{len(self._errors)} trajectory log writes failed") from self._errors[0]

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()
