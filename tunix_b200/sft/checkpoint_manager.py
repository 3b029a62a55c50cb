"""Checkpoint save / restore with the directory layout of the reference's Orbax checkpoints.

Layout (tunix/sft/checkpoint_manager.py:124-358, fixture tests/sft/test_data/checkpoints/1/):

    <root>/<step>/_CHECKPOINT_METADATA           JSON, includes `custom_metadata`
    <root>/<step>/model_params/_METADATA         JSON tree: "('layers', '0', 'weight')" -> array info
    <root>/<step>/model_params/<dotted.name>/.zarray + 0   zarr-v2 array, one chunk, raw little-endian bytes
    <root>/<step>/optimizer_state/...            same, keys ('mu'|'nu'|'master', <param name>)

Arrays are written as plain (non-OCDBT) zarr-v2 chunk files; bfloat16 uses dtype string "bfloat16"
with the raw 2-byte payload. A parameter `layers.0.weight` is recorded in `_METADATA` under the key tuple
('layers', '0', 'weight') and stored in the directory `layers.0.weight`, which is how Orbax names the arrays
of a nested tree. LoRA models save / restore adapter parameters only (partial restore).
Saves run on a background thread after a device->host copy (async checkpointing); policies:
fixed step interval or "at least N seconds since the last save", keep the latest `max_to_keep`.
`maybe_restore` returns `(step, custom_metadata)`.

Reading: `_load_item` also reads item directories that Orbax wrote in its OCDBT layout (`sft/ocdbt.py`; checked
against a checkpoint written by the reference's own test suite). Writing stays plain zarr-v2 directories per array,
the non-OCDBT form of the same layout; whether Orbax accepts them has not been checked here (Orbax is not
installable offline).

Several ranks: the decision to save is taken on rank 0 and broadcast (a wall-clock policy would otherwise let
ranks disagree and hang the collectives below); every rank then takes part in gathering sharded state (a
sharded optimizer's `state_dict()`, parameters that carry `shard_spec = (dim, index, count)` from the tensor /
weight / expert parallel modules) so that the arrays written are whole tensors under their full names; only
rank 0 touches the file system. On restore every rank reads the whole array and keeps its own slice.
"""
from __future__ import annotations

import json
import os
import shutil
import threading
import time
from typing import Any, Optional

import numpy as np
import torch

from ..common.configs import CheckpointingOptions

_DT = {torch.float32: "<f4", torch.float16: "<f2", torch.bfloat16: "bfloat16", torch.int32: "<i4",
       torch.int64: "<i8", torch.uint8: "|u1", torch.int8: "|i1", torch.bool: "|b1", torch.float64: "<f8",
       torch.int16: "<i2"}
_DT_INV = {v: k for k, v in _DT.items()}


def _write_array(path: str, t: torch.Tensor) -> dict:
    os.makedirs(path, exist_ok=True)
    t = t.detach().contiguous().cpu()
    meta = {"zarr_format": 2, "shape": list(t.shape), "chunks": list(t.shape) or [1], "dtype": _DT[t.dtype],
            "compressor": None, "fill_value": 0, "order": "C", "filters": None}
    with open(os.path.join(path, ".zarray"), "w") as f:
        json.dump(meta, f)
    raw = t.view(torch.uint8).numpy() if t.dtype != torch.bool else t.to(torch.uint8).numpy()
    chunk_name = ".".join(["0"] * max(t.dim(), 1))
    with open(os.path.join(path, chunk_name), "wb") as f:
        f.write(raw.tobytes())
    return {"shape": list(t.shape), "dtype": _DT[t.dtype]}


def _read_array(path: str) -> torch.Tensor:
    with open(os.path.join(path, ".zarray")) as f:
        meta = json.load(f)
    dt = _DT_INV[meta["dtype"]]
    shape = meta["shape"]
    chunk_name = ".".join(["0"] * max(len(shape), 1))
    with open(os.path.join(path, chunk_name), "rb") as f:
        raw = np.frombuffer(f.read(), dtype=np.uint8).copy()
    t = torch.from_numpy(raw)
    if dt == torch.bool:
        return t.view(torch.uint8).bool().view(shape)
    return t.view(dt).view(shape)


def _flatten(tree: Any, prefix=()) -> dict:
    out = {}
    if isinstance(tree, dict):
        for k, v in tree.items():
            out.update(_flatten(v, prefix + (str(k),)))
    else:
        out[prefix] = tree
    return out


def _split_keys(tree: Any) -> Any:
    """{'a.b.c': t} -> {'a': {'b': {'c': t}}}: dotted parameter names become the nested tree Orbax would see."""
    if not isinstance(tree, dict):
        return tree
    out: dict = {}
    for k, v in tree.items():
        parts = str(k).split(".")
        d = out
        for part in parts[:-1]:
            d = d.setdefault(part, {})
            if not isinstance(d, dict):
                raise ValueError(f"checkpoint key {k!r} is both a leaf and a prefix of another key")
        if isinstance(d.get(parts[-1]), dict):
            raise ValueError(f"checkpoint key {k!r} is both a leaf and a prefix of another key")
        d[parts[-1]] = _split_keys(v)
    return out


def _dist():
    import torch.distributed as dist
    return dist if (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1) else None


def _gather_sharded(t: torch.Tensor, owner) -> torch.Tensor:
    """Whole tensor from the slices that the ranks of `owner.shard_group` hold along `owner.shard_spec[0]`.
    Collective over that group; a tensor without a `shard_spec` comes back as it is."""
    spec = getattr(owner, "shard_spec", None)
    dist = _dist()
    if spec is None or dist is None or spec[2] <= 1:
        return t
    dim, _, count = spec
    group = getattr(owner, "shard_group", None)
    t = t.detach().contiguous()
    parts = [torch.empty_like(t) for _ in range(count)]
    dist.all_gather(parts, t, group=group)
    return torch.cat(parts, dim=dim)


def _slice_for(t: torch.Tensor, owner) -> torch.Tensor:
    spec = getattr(owner, "shard_spec", None)
    if spec is None or spec[2] <= 1 or tuple(t.shape) == tuple(owner.shape):
        return t
    dim, index, count = spec
    n = t.shape[dim] // count
    return t.narrow(dim, index * n, n)


def _save_item(path: str, tree: dict) -> None:
    os.makedirs(path, exist_ok=True)
    flat = _flatten(_split_keys(tree))
    md = {}
    for key, val in flat.items():
        name = ".".join(key)
        if isinstance(val, torch.Tensor):
            info = _write_array(os.path.join(path, name), val)
            md[str(key)] = {"key_metadata": [{"key": k, "key_type": 2} for k in key],
                            "value_metadata": {"value_type": "jax.Array", "skip_deserialize": False, **info}}
        else:
            md[str(key)] = {"key_metadata": [{"key": k, "key_type": 2} for k in key],
                            "value_metadata": {"value_type": "scalar", "value": val}}
    with open(os.path.join(path, "_METADATA"), "w") as f:
        json.dump({"tree_metadata": md, "use_zarr3": False}, f)


def _load_item(path: str) -> dict:
    if os.path.exists(os.path.join(path, "manifest.ocdbt")):
        # written by Orbax itself in its OCDBT layout: arrays packed into a B+tree key-value store (`sft/ocdbt.py`)
        from . import ocdbt
        out: dict = {}
        for key, arr in ocdbt.load_tree(path).items():
            d = out
            for k in key[:-1]:
                d = d.setdefault(k, {})
            d[key[-1]] = torch.from_numpy(np.ascontiguousarray(arr))
        return out
    with open(os.path.join(path, "_METADATA")) as f:
        md = json.load(f)["tree_metadata"]
    out: dict = {}
    for skey, info in md.items():
        key = tuple(k["key"] for k in info["key_metadata"])
        vm = info["value_metadata"]
        val = _read_array(os.path.join(path, ".".join(key))) if vm["value_type"] == "jax.Array" else vm["value"]
        d = out
        for k in key[:-1]:
            d = d.setdefault(k, {})
        d[key[-1]] = val
    return out


class CheckpointManager:
    def __init__(self, root_directory: Optional[str] = None, options: Any = None, group=None):
        """`group`: the process group of the ranks that train this model (None = every rank of the job). Decisions
        are taken by, and files written by, the group's first rank; the collectives of this class stay inside the
        group, so ranks that host other roles (samplers of a disaggregated RL job) are not involved."""
        self._root = root_directory
        self._group = group
        if isinstance(options, dict) or options is None:
            options = CheckpointingOptions.from_dict(options)
        self._opts: CheckpointingOptions = options
        self._last_save_time = time.time()
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        self._decisions: dict = {}
        if self._root:
            os.makedirs(self._root, exist_ok=True)

    # ------------------------------------------------------------------ queries
    def all_steps(self) -> list[int]:
        if not self._root or not os.path.isdir(self._root):
            return []
        steps = []
        for d in os.listdir(self._root):
            if d.isdigit() and os.path.exists(os.path.join(self._root, d, "_CHECKPOINT_METADATA")):
                steps.append(int(d))
        return sorted(steps)

    def latest_step(self) -> Optional[int]:
        s = self.all_steps()
        return s[-1] if s else None

    def _should_save(self, step: int, force: bool) -> bool:
        if not self._root:
            return False
        if force:
            return step not in self.all_steps()
        o = self._opts
        if o.save_interval_steps:
            return step % o.save_interval_steps == 0
        if o.save_interval_secs is not None:
            return time.time() - self._last_save_time >= o.save_interval_secs
        return False

    def should_save(self, step: int, force: bool = False) -> bool:
        """The decision for `step`, the same on every rank: rank 0 decides (its clock, its view of the directory)
        and the others are told, because the gathers inside `save` are collectives."""
        if not self._root:
            return False
        cached = self._decisions.get((step, force))
        if cached is not None:
            return cached
        dist = _dist()
        if dist is None:
            decision = self._should_save(step, force)
        else:
            box = [self._should_save(step, force) if self._is_writer() else None]
            dist.broadcast_object_list(box, src=self._src(), group=self._group)
            decision = bool(box[0])
        self._decisions = {(step, force): decision}
        return decision

    def _src(self) -> int:
        """Global rank of the rank that decides and writes."""
        dist = _dist()
        if dist is None or self._group is None:
            return 0
        return dist.get_global_rank(self._group, 0)

    def _is_writer(self) -> bool:
        dist = _dist()
        return dist is None or dist.get_rank() == self._src()

    # --------------------------------------------------------------------- save
    def save(self, step: int, model, optimizer=None, save_only_lora_params: bool = False, force: bool = False,
             custom_metadata: Optional[dict] = None) -> bool:
        if not self.should_save(step, force):
            return False
        self._decisions = {}
        self.wait_until_finished()
        from ..lora import is_lora_param_name
        writer = self._is_writer()
        # Collective part (every rank): whole tensors out of sharded ones. Device -> host copies happen here
        # (synchronously) on the rank that writes; file IO on its worker thread.
        owners = dict(model.named_parameters())
        params = {}
        for n, p in owners.items():
            if save_only_lora_params and not is_lora_param_name(n):
                continue
            full = _gather_sharded(p.detach(), p)
            if writer:
                params[n] = full.to("cpu", copy=True)
        opt_state = None
        if optimizer is not None:
            sd = optimizer.state_dict()           # a sharded optimizer gathers here, on every rank
            opt_state = {}
            for k, v in sd.items():
                if isinstance(v, dict):
                    d = {}
                    for n, t in v.items():
                        full = _gather_sharded(t.detach(), owners.get(n))
                        if writer:
                            d[n] = full.to("cpu", copy=True)
                    opt_state[k] = d
                else:
                    opt_state[k] = v
        self._last_save_time = time.time()
        if not writer:
            return True
        meta = {"step": step, "custom_metadata": custom_metadata or {}, "init_timestamp_nsecs": time.time_ns(),
                "item_handlers": {"model_params": "StandardCheckpointHandler",
                                  "optimizer_state": "StandardCheckpointHandler"}}

        def work():
            try:
                tmp = os.path.join(self._root, f"{step}.orbax-checkpoint-tmp")
                final = os.path.join(self._root, str(step))
                shutil.rmtree(tmp, ignore_errors=True)
                os.makedirs(tmp)
                _save_item(os.path.join(tmp, "model_params"), params)
                if opt_state is not None:
                    _save_item(os.path.join(tmp, "optimizer_state"), opt_state)
                meta["commit_timestamp_nsecs"] = time.time_ns()
                with open(os.path.join(tmp, "_CHECKPOINT_METADATA"), "w") as f:
                    json.dump(meta, f)
                shutil.rmtree(final, ignore_errors=True)
                os.replace(tmp, final)
                self._apply_retention()
            except BaseException as e:  # surfaced on the next wait
                self._error = e

        if self._opts.enable_async_checkpointing:
            self._thread = threading.Thread(target=work, name="ckpt-save", daemon=True)
            self._thread.start()
        else:
            work()
            self._raise_pending()
        return True

    def _apply_retention(self) -> None:
        keep = self._opts.max_to_keep
        if not keep:
            return
        steps = self.all_steps()
        for s in steps[:-keep]:
            shutil.rmtree(os.path.join(self._root, str(s)), ignore_errors=True)

    def _raise_pending(self):
        if self._error is not None:
            e, self._error = self._error, None
            raise RuntimeError("checkpoint save failed") from e

    def wait_until_finished(self) -> None:
        if self._thread is not None:
            self._thread.join(self._opts.timeout_secs)
            if self._thread.is_alive():
                raise TimeoutError("checkpoint save did not finish in time")
            self._thread = None
        self._raise_pending()

    # ------------------------------------------------------------------ restore
    def maybe_restore(self, model, optimizer=None, step: Optional[int] = None, restore_only_lora_params: bool = False):
        """Restore the latest (or given) step in place. Returns (step, custom_metadata); (0, {}) if none."""
        if not self._root:
            return 0, {}
        self.wait_until_finished()
        dist = _dist()
        if dist is not None:
            dist.barrier(group=self._group)              # the writing rank has finished its last save
            if step is None:
                box = [self.latest_step() if self._is_writer() else None]
                dist.broadcast_object_list(box, src=self._src(), group=self._group)
                step = box[0]
        step = self.latest_step() if step is None else step
        if step is None:
            return 0, {}
        d = os.path.join(self._root, str(step))
        with open(os.path.join(d, "_CHECKPOINT_METADATA")) as f:
            meta = json.load(f)
        from ..lora import is_lora_param_name
        saved = _flatten(_load_item(os.path.join(d, "model_params")))
        saved = {".".join(k): v for k, v in saved.items()}
        with torch.no_grad():
            for n, p in model.named_parameters():
                if restore_only_lora_params and not is_lora_param_name(n):
                    continue
                if n in saved:
                    p.copy_(_slice_for(saved[n], p).to(p.device, p.dtype))
                elif not restore_only_lora_params and not saved_is_partial(saved):
                    raise KeyError(f"parameter {n} missing from checkpoint {d}")
        if optimizer is not None and os.path.isdir(os.path.join(d, "optimizer_state")):
            sd = _load_item(os.path.join(d, "optimizer_state"))
            fixed = {}
            owners = dict(model.named_parameters())
            unsharded_state = getattr(optimizer, "is_sharded", False)   # it slices whole tensors itself
            for k, v in sd.items():
                if isinstance(v, dict):
                    fixed[k] = {".".join(kk): (vv if unsharded_state or ".".join(kk) not in owners
                                               else _slice_for(vv, owners[".".join(kk)]))
                                for kk, vv in _flatten(v).items()}
                else:
                    fixed[k] = v
            optimizer.load_state_dict(fixed)
        return int(meta.get("step", step)), meta.get("custom_metadata", {}) or {}

    def close(self) -> None:
        self.wait_until_finished()


def saved_is_partial(saved: dict) -> bool:
    from ..lora import is_lora_param_name
    return bool(saved) and all(is_lora_param_name(n) for n in saved)
