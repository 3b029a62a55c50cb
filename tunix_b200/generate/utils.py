"""Sampler-side helpers and the name-mapped weight transfer (tunix/generate/utils.py:35-2278).

Three groups:

* token bookkeeping for samplers (:87-340, :2116-2278): padding, first / last non-pad positions, first EOS, prompt
  rows from strings or token ids, left padding to a bucket length, the check that an engine echoed the prompts it
  was given, conflicting sampling options;
* `transfer_state_with_mappings` (:361-1006): copy a trainer's parameters into a differently named / laid out
  rollout model: `*` wildcards over layer indices, source tensors stacked over layers, transposes, per-key hooks,
  shape alignment (reshape, zero-padded head dim, repeated kv heads), dtype cast, tied lm_head, and an optional
  reshard step run in bounded chunks (:1595-1668);
* mixture-of-experts layout helpers (:1258-1510): gate / up projections fused per shard, plain or interleaved in
  lanes; `verify_state_closeness` (:2040-2092) and `resolve_parallelism_sizes` (:1996-2037).

States are plain `{name: tensor}` dicts (a module's `state_dict()` or `dict(named_parameters())`); tuple keys are
joined with dots.
"""
from __future__ import annotations

import logging
import math
import re
from typing import Any, Callable, Mapping, Optional, Sequence

import numpy as np
import torch

log = logging.getLogger(__name__)


# ------------------------------------------------------------------------------------------ small arithmetic
def next_power_of_2(x: int) -> int:
    if x <= 0:
        raise ValueError("next_power_of_2 needs a positive integer")
    return 1 << (int(x) - 1).bit_length()


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def pad_to_length(x, target_length: int, pad_value=0, left: bool = False, axis: int = 0):
    """Pad a numpy array or tensor along `axis` up to `target_length` (longer inputs come back unchanged)."""
    n = x.shape[axis]
    if n >= target_length:
        return x
    if isinstance(x, torch.Tensor):
        shape = list(x.shape)
        shape[axis] = target_length - n
        fill = torch.full(shape, pad_value, dtype=x.dtype, device=x.device)
        return torch.cat([fill, x] if left else [x, fill], dim=axis)
    widths = [(0, 0)] * x.ndim
    widths[axis] = (target_length - n, 0) if left else (0, target_length - n)
    return np.pad(x, widths, constant_values=pad_value)


def find_first_non_pad_idx(ids, pad_id: int) -> int:
    """Index of the first token that is not padding (0 when the row is all padding)."""
    a = np.asarray(ids.cpu() if isinstance(ids, torch.Tensor) else ids)
    nz = np.flatnonzero(a != pad_id)
    return int(nz[0]) if nz.size else 0


def find_last_non_pad_idx(ids, pad_id: int) -> int:
    """Index of the last token that is not padding (-1 when the row is all padding)."""
    a = np.asarray(ids.cpu() if isinstance(ids, torch.Tensor) else ids)
    nz = np.flatnonzero(a != pad_id)
    return int(nz[-1]) if nz.size else -1


def find_first_eos_idx(ids, eos_id) -> int:
    """Index of the first end-of-sequence token (any of `eos_id` when several are given); len(ids) when none."""
    a = np.asarray(ids.cpu() if isinstance(ids, torch.Tensor) else ids)
    hit = np.isin(a, np.atleast_1d(np.asarray(eos_id)))
    nz = np.flatnonzero(hit)
    return int(nz[0]) if nz.size else int(a.shape[0])


def build_positions_from_mask(input_mask: torch.Tensor) -> torch.Tensor:
    """Positions that count real tokens only: cumsum(mask) - 1, clamped at 0 over the left padding."""
    m = input_mask.to(torch.int64)
    return (torch.cumsum(m, dim=-1) - 1).clamp(min=0)


def make_causal_attn_mask(input_mask: torch.Tensor, cache_size: Optional[int] = None) -> torch.Tensor:
    """[B, T, S] boolean mask: token t sees the real tokens at or before it; S = cache_size pads the key side."""
    B, T = input_mask.shape
    S = cache_size or T
    causal = torch.tril(torch.ones(T, S, dtype=torch.bool, device=input_mask.device))
    keys = torch.zeros(B, S, dtype=torch.bool, device=input_mask.device)
    keys[:, :T] = input_mask.bool()
    return causal[None] & keys[:, None, :]


def check_sampling_mode_conflict(original_mode: list, new_mode: str) -> None:
    """A sampler call picks one of greedy / top-p / beam search; naming a second one is an error."""
    if original_mode[0] is not None and original_mode[0] != new_mode:
        raise ValueError(f"Conflicting sampling modes: {original_mode[0]!r} was selected, {new_mode!r} asked for as well")
    original_mode[0] = new_mode


# ------------------------------------------------------------------------------------------------ prompt rows
def is_token_id_sequence(prompt: Any) -> bool:
    """True for a 1-D integer array or a non-empty list / tuple of ints."""
    if isinstance(prompt, np.ndarray):
        return prompt.ndim == 1 and np.issubdtype(prompt.dtype, np.integer)
    if isinstance(prompt, torch.Tensor):
        return prompt.dim() == 1 and not prompt.dtype.is_floating_point
    return isinstance(prompt, (list, tuple)) and len(prompt) > 0 and isinstance(prompt[0], (int, np.integer))


def as_token_ids(value) -> np.ndarray:
    """An owned 1-D int32 copy of a row of token ids."""
    if isinstance(value, torch.Tensor):
        value = value.detach().cpu().numpy()
    arr = np.array(value, dtype=np.int32)
    if arr.ndim != 1:
        raise ValueError(f"token ids must be 1-D, got shape {arr.shape}")
    return arr


def unpad_prompt(padded_tokens, length: int) -> np.ndarray:
    """The last `length` tokens of a left-padded row."""
    arr = as_token_ids(padded_tokens)
    return arr[-int(length):] if length > 0 else np.zeros(0, np.int32)


def unpad_prompt_tokens(padded_tokens, pad_id: Optional[int] = None, prompt_length: Optional[int] = None) -> np.ndarray:
    """A prompt row without its left padding: by its known length, else by the first token that is not `pad_id`."""
    if prompt_length is not None:
        return unpad_prompt(padded_tokens, int(prompt_length))
    arr = as_token_ids(np.asarray(padded_tokens).reshape(-1))
    if pad_id is None:
        return arr
    nz = np.flatnonzero(arr != pad_id)
    return arr[nz[0]:] if nz.size else np.zeros(0, np.int32)


def resolve_prompt_tokens(input_strings, prompt_token_ids, tokenize_fn: Callable[[str], Any], *,
                          max_generation_steps: int = 0, max_total_length: Optional[int] = None,
                          max_length_name: str = "max_model_len", single_output_per_row: bool = True) -> list:
    """Token rows from exactly one of `input_strings` / `prompt_token_ids`, with the length budget checked for rows
    given as ids (strings are truncated by the tokenizer's caller)."""
    if (input_strings is None) == (prompt_token_ids is None):
        raise ValueError("Provide exactly one of input_strings or prompt_token_ids")
    if prompt_token_ids is not None:
        if len(prompt_token_ids) == 0:
            raise ValueError("prompt_token_ids must not be empty")
        if not single_output_per_row:
            raise ValueError("prompt_token_ids requires exactly one output per row")
        rows = [as_token_ids(r) for r in prompt_token_ids]
        if max_total_length is not None and any(len(r) + max_generation_steps > max_total_length for r in rows):
            raise ValueError(f"prompt plus max_generation_steps exceeds {max_length_name}")
        return rows
    if isinstance(input_strings, np.ndarray):
        input_strings = input_strings.tolist()
    if isinstance(input_strings, str):
        input_strings = [input_strings]
    if len(input_strings) == 0:
        raise ValueError("input_strings must not be empty")
    return [np.asarray(tokenize_fn(str(s)), dtype=np.int32) for s in input_strings]


def left_pad_prompt_tokens(prompt_ids: Sequence, max_prompt_length: Optional[int], pad_value: int, *,
                           max_allowed_length: Optional[int] = None):
    """(ids [B, L] left padded, lengths [B], L). L is `max_prompt_length` when it fits the longest row, else the next
    power of two above it (capped by `max_allowed_length` when the longest row still fits under the cap)."""
    lengths = np.array([len(r) for r in prompt_ids], dtype=np.int32)
    longest = int(lengths.max())
    if max_prompt_length is None or max_prompt_length < longest:
        max_prompt_length = next_power_of_2(longest)
        if max_allowed_length is not None and longest <= max_allowed_length:
            max_prompt_length = min(max_prompt_length, max_allowed_length)
    ids = np.stack([pad_to_length(np.asarray(r, np.int32), max_prompt_length, pad_value, left=True) for r in prompt_ids])
    return ids.astype(np.int32), lengths, int(max_prompt_length)


def _field(obj, key, default=None):
    return obj.get(key, default) if isinstance(obj, dict) else getattr(obj, key, default)


def check_prompt_echo(expected_ids: Sequence[np.ndarray], outputs: Sequence[Any], *, backend_name: str = "Engine") -> None:
    """An engine that was handed token rows must answer with one output per row, distinct request ids, and the same
    prompt tokens (or at least their count); anything else means rows were dropped, merged or re-tokenised."""
    if len(outputs) != len(expected_ids):
        raise ValueError(f"{backend_name} result count differs from submitted token rows: expected {len(expected_ids)}, "
                         f"got {len(outputs)}")
    seen = set()
    for want, out in zip(expected_ids, outputs):
        meta = _field(out, "meta_info") or {}
        rid = _field(out, "request_id", _field(meta, "id"))
        if rid is None:
            raise ValueError(f"{backend_name} output is missing request_id")
        if rid in seen:
            raise ValueError(f"{backend_name} returned duplicate request ids (duplicate request_id: {rid})")
        seen.add(rid)
        echoed = _field(out, "prompt_token_ids", _field(meta, "prompt_tokens"))
        if echoed is None:
            raise ValueError(f"{backend_name} output is missing prompt echo / prompt_token_ids")
        same = int(echoed) == len(want) if isinstance(echoed, (int, np.integer)) else np.array_equal(as_token_ids(echoed), want)
        if not same:
            raise ValueError(f"{backend_name} prompt echo / prompt_token_ids differed from input")


def resolve_parallelism_sizes(mesh, tensor_parallel_size: int = -1, data_parallel_size: int = -1,
                              expert_parallel_size: int = 1):
    """(tp, dp, ep) with -1 entries inferred from the number of ranks of `mesh` (an object with `.shape` as a dict or
    tuple, or a plain rank count). With both tp and dp unknown everything that is not ep becomes tp."""
    shape = getattr(mesh, "shape", mesh)
    total = int(shape) if isinstance(shape, (int, np.integer)) else math.prod(shape.values() if isinstance(shape, Mapping) else shape)
    if total % expert_parallel_size:
        raise ValueError(f"Total mesh devices ({total}) must be divisible by expert_parallel_size ({expert_parallel_size}).")
    if tensor_parallel_size == -1 and data_parallel_size == -1:
        tensor_parallel_size, data_parallel_size = total // expert_parallel_size, 1
    elif tensor_parallel_size == -1:
        tensor_parallel_size = total // (data_parallel_size * expert_parallel_size)
    elif data_parallel_size == -1:
        data_parallel_size = total // (tensor_parallel_size * expert_parallel_size)
    return tensor_parallel_size, data_parallel_size, expert_parallel_size


# --------------------------------------------------------------------------------- name-mapped weight transfer
class ShapeMismatchError(ValueError):
    """A source tensor cannot be brought to its target's shape by reshape, head-dim padding or head repetition."""


class MappingError(ValueError):
    """A target parameter has no source, or a mapped source is absent."""


def _flat(state) -> dict:
    if hasattr(state, "state_dict"):
        state = state.state_dict()
    return {(".".join(str(k) for k in key) if isinstance(key, (tuple, list)) else str(key)): v for key, v in state.items()}


def build_flat_dict(dst_names: Sequence[str], mappings: Mapping[str, tuple]) -> dict:
    """{source name: (target names, layout)} for every target that some mapping produces.

    `mappings`: source pattern -> (target pattern, layout). A `*` path component stands for a layer index and must
    appear on both sides; a target pattern may instead be a regular expression (it then contains `|` or parentheses)
    whose groups fill the source's `*`s in order. A layout that names a "layer" axis (a tuple containing the string
    "layer") marks a source STACKED over layers: all matching targets are collected, sorted by layer, under the one
    source name, and the stacked tensor is split along that axis. Targets without a mapping are reported once."""
    compiled = []
    for src, (tgt, layout) in mappings.items():
        if any(c in tgt for c in "|()"):
            pat = "^" + tgt + "$"
        else:
            pat = "^" + re.escape(tgt).replace(r"\.\*", r"\.(\d+)").replace(r"\*\.", r"(\d+)\.") + "$"
        compiled.append((src, re.compile(pat), layout))
    out, unmapped = {}, []
    for name in dst_names:
        for src, rx, layout in compiled:
            m = rx.match(name)
            if not m:
                continue
            groups = iter(m.groups())
            stacked = layout is not None and "layer" in tuple(layout)
            parts = []
            for part in src.split("."):
                if part == "*" and not stacked:
                    parts.append(next(groups))
                elif part != "*":
                    parts.append(part)
            actual = ".".join(parts)
            if stacked:
                layer = int(m.groups()[0]) if m.groups() else 0
                out.setdefault(actual, ([], layout))[0].append((layer, name))
            else:
                out[actual] = ([(0, name)], layout)
            break
        else:
            unmapped.append(name)
    if unmapped:
        log.warning("no mapping for target parameters: %s", unmapped)
    return {k: ([n for _, n in sorted(v[0])], v[1]) for k, v in out.items()}


def _repeat_to(val: torch.Tensor, dim: int, size: int, key: str) -> torch.Tensor:
    if size % val.shape[dim]:
        raise ShapeMismatchError(f"{key}: cannot repeat {val.shape[dim]} heads to {size}")
    return val.repeat_interleave(size // val.shape[dim], dim=dim)


def align_shape(val: torch.Tensor, tgt_shape: tuple, key: str = "", *, num_kv_heads: Optional[int] = None,
                head_dim: Optional[int] = None) -> torch.Tensor:
    """Bring `val` to `tgt_shape`:

    * equal element counts: reshape (a [D, N, H] projection against a [D, N*H] target, a flat bias against [N, H]);
    * same rank, some dims smaller: zero-pad a head dim (the trailing axis of q / k / v projections, the axis
      before last of an output projection) and REPEAT a kv-head axis that the target replicates (a rollout engine
      that runs more tensor-parallel ranks than there are kv heads);
    * a flat kv bias [K*H] against [K', H] with K' a multiple of K: reshape, then repeat heads (needs
      `num_kv_heads` and `head_dim`)."""
    tgt_shape = tuple(tgt_shape)
    if tuple(val.shape) == tgt_shape:
        return val
    if val.numel() == math.prod(tgt_shape):
        return val.reshape(tgt_shape)
    if val.dim() != len(tgt_shape):
        if val.dim() == 1 and len(tgt_shape) == 2 and num_kv_heads and head_dim and val.shape[0] == num_kv_heads * head_dim \
                and tgt_shape[1] == head_dim:
            return _repeat_to(val.reshape(num_kv_heads, head_dim), 0, tgt_shape[0], key)
        raise ShapeMismatchError(f"{key}: rank {val.dim()} {tuple(val.shape)} against {tgt_shape}")
    is_out_proj = "o_proj" in key or "attn_vec" in key
    head_axis = val.dim() - 2 if is_out_proj else val.dim() - 1          # where a head dim may be padded
    for ax, (s, t) in enumerate(zip(val.shape, tgt_shape)):
        if s == t:
            continue
        if s > t:
            raise ShapeMismatchError(f"{key}: axis {ax} shrinks from {s} to {t}")
        if ax == head_axis and val.dim() >= 3:
            pad = [0, 0] * val.dim()
            pad[2 * (val.dim() - 1 - ax) + 1] = t - s
            val = torch.nn.functional.pad(val, pad)
        else:
            val = _repeat_to(val, ax, t, key)
    return val


def _sync_tied_lm_head(dst: dict, written: set) -> None:
    """A target that materialises `lm_head` although the source ties it to the embedding gets the embedding."""
    heads = [k for k in dst if k.endswith("lm_head") or k.endswith("lm_head.weight")]
    embeds = [k for k in dst if "embed_tokens" in k or k.endswith("embedder.input_embedding")]
    for h in heads:
        if h not in written and embeds and dst[embeds[0]].shape == dst[h].shape:
            dst[h].copy_(dst[embeds[0]])
            written.add(h)


def reshard_in_chunks(values: dict, specs: dict, reshard_fn: Callable[[dict, dict], dict], chunk_size: int) -> dict:
    """Run `reshard_fn` over at most `chunk_size` bytes of tensors at a time, so that the staging memory of a
    cross-rank transfer is bounded by the chunk instead of by the model (tunix/generate/utils.py:1595-1668)."""
    out, batch, size = {}, {}, 0
    for k, v in values.items():
        nbytes = v.numel() * v.element_size()
        if batch and size + nbytes > chunk_size:
            out.update(reshard_fn(batch, {b: specs.get(b) for b in batch}))
            batch, size = {}, 0
        batch[k] = v
        size += nbytes
    if batch:
        out.update(reshard_fn(batch, {b: specs.get(b) for b in batch}))
    return out


@torch.no_grad()
def transfer_state_with_mappings(src_state, dst_state, key_mappings: Mapping[str, tuple], key_mapping_hook_fns=None,
                                 transpose_keys: Optional[Mapping[str, tuple]] = None, reshard_fn=None,
                                 rollout_engine: Optional[str] = None, **kwargs) -> dict:
    """Write the source parameters into the target's tensors (in place) following `key_mappings`
    (see `build_flat_dict`). Per source tensor, in this order: split along the layer axis when stacked; transpose
    (`transpose_keys`: a key's last path component or full name -> permutation); per-key hook; `align_shape`; cast to
    the target's dtype. `reshard_fn(values, specs)` (with `reshard_chunk_size=` bytes to run it in chunks) lets the
    caller place the converted tensors (for instance a cross-rank `WeightReshard`); without it values are copied into
    the target tensors directly. Returns the target dict."""
    src, dst = _flat(src_state), _flat(dst_state)
    plan = build_flat_dict(list(dst), key_mappings)
    converted, written = {}, set()
    for src_key, (tgt_names, layout) in plan.items():
        if src_key not in src:
            raise MappingError(f"mapped source {src_key!r} is not in the source state")
        val = src[src_key]
        if layout is not None and "layer" in tuple(layout):
            axis = tuple(layout).index("layer")
            if val.shape[axis] != len(tgt_names):
                raise ShapeMismatchError(f"{src_key}: {val.shape[axis]} stacked layers against {len(tgt_names)} targets")
            pieces = list(val.unbind(axis))
        else:
            pieces = [val]
        for piece, name in zip(pieces, tgt_names):
            if transpose_keys:
                perm = transpose_keys.get(src_key, transpose_keys.get(src_key.rsplit(".", 1)[-1]))
                if perm is not None and len(perm) == piece.dim():
                    piece = piece.permute(*perm)
            if key_mapping_hook_fns and src_key in key_mapping_hook_fns:
                piece = key_mapping_hook_fns[src_key](piece)
            tgt = dst[name]
            piece = align_shape(piece, tuple(tgt.shape), src_key, num_kv_heads=kwargs.get("num_kv_heads"),
                                head_dim=kwargs.get("head_dim"))
            converted[name] = piece.to(tgt.dtype)
            written.add(name)
    if reshard_fn is not None:
        specs = {k: getattr(dst[k], "shard_spec", None) for k in converted}
        chunk = kwargs.get("reshard_chunk_size")
        placed = reshard_in_chunks(converted, specs, reshard_fn, chunk) if chunk else reshard_fn(converted, specs)
        for k, v in placed.items():
            if v is not dst[k]:
                dst[k].copy_(v)
    else:
        for k, v in converted.items():
            dst[k].copy_(v)
    _sync_tied_lm_head(dst, written)
    return dst


def verify_state_closeness(golden_state, state, atol: float = 1e-2) -> bool:
    """True when both states have the same names and shapes and every tensor agrees within `atol`; differences are
    logged with the first values of both sides."""
    a, b = _flat(golden_state), _flat(state)
    if a.keys() != b.keys():
        log.info("keys differ; missing %s, extra %s", set(a) - set(b), set(b) - set(a))
        return False
    ok = True
    for k in a:
        if a[k].shape != b[k].shape:
            log.info("shape mismatch for %s: golden %s, loaded %s", k, tuple(a[k].shape), tuple(b[k].shape))
            ok = False
        elif not torch.allclose(a[k].float(), b[k].float().to(a[k].device), atol=atol, rtol=0.0):
            log.info("weights for %s differ: golden %s loaded %s", k, a[k].flatten()[:10].tolist(), b[k].flatten()[:10].tolist())
            ok = False
    return ok


# ------------------------------------------------------------------------------------- mixture-of-experts layouts
def interleave_moe_weights(gate: torch.Tensor, up: torch.Tensor, tgt_shape: tuple, n_shards: int = 1,
                           axis: Optional[int] = None, lane_size: int = 0) -> torch.Tensor:
    """One fused gate / up tensor of `tgt_shape` from separate `gate` and `up` projections
    (tunix/generate/utils.py:1258-1318). Along `axis` (default: last) the target holds, for each of `n_shards`
    tensor-parallel shards, that shard's gate columns followed by its up columns, each zero-padded to the target's
    per-shard width; with `lane_size > 0` (and a per-shard width divisible by it) gate and up alternate in blocks of
    `lane_size` columns inside the shard instead."""
    nd = len(tgt_shape)
    axis = nd - 1 if axis is None else axis % nd
    half = tgt_shape[axis] // 2
    per_shard = half // n_shards

    def chunks(t):
        own = t.shape[axis] // n_shards
        shp = list(t.shape)
        shp[axis:axis + 1] = [n_shards, own]
        t = t.reshape(shp)
        if per_shard > own:
            pad = [0, 0] * t.dim()
            pad[2 * (t.dim() - 1 - (axis + 1)) + 1] = per_shard - own
            t = torch.nn.functional.pad(t, pad)
        return t

    g, u = chunks(gate), chunks(up)
    if lane_size and per_shard % lane_size == 0:
        shp = list(g.shape)
        shp[axis + 1:axis + 2] = [per_shard // lane_size, lane_size]
        both = torch.stack([g.reshape(shp), u.reshape(shp)], dim=axis + 2)
    else:
        both = torch.cat([g, u], dim=axis + 1)
    return both.reshape(tgt_shape)


def fuse_moe_weights(src: dict, dst: dict, *, gate_name: str = "wi_0", up_name: str = "wi_1", fused_name: str = "wi",
                     n_shards: int = 1, lane_size: int = 0) -> dict:
    """A copy of `src` in which every `<prefix>.<gate_name>` / `<prefix>.<up_name>` pair whose target holds
    `<prefix>.<fused_name>` is replaced by the fused tensor in the target's shape (tunix/generate/utils.py:1455-1510).
    The fused axis is the last one on which source and target differ."""
    out = dict(_flat(src))
    for name, tgt in _flat(dst).items():
        if not name.endswith("." + fused_name) and name != fused_name:
            continue
        prefix = name[: -len(fused_name)]
        g, u = out.get(prefix + gate_name), out.get(prefix + up_name)
        if g is None or u is None:
            continue
        diff = [i for i, (s, t) in enumerate(zip(g.shape, tgt.shape)) if s != t]
        axis = diff[-1] if diff else len(tgt.shape) - 1
        del out[prefix + gate_name], out[prefix + up_name]
        out[name] = interleave_moe_weights(g, u, tuple(tgt.shape), n_shards, axis=axis, lane_size=lane_size)
    return out
