"""Sequence packing for RL train batches: dataclasses, the native (C++) fast path and a Python twin.

`PackItem` / `PackedRow` / `PackedChunk` carry the same fields as the reference
(tunix/rl/packing.py:60-222). `fill_one_chunk` (FFD assignment), `pack_chunk` (row fill) and
`pack_core` (multi-chunk loop) call `libtunix_b200_host.so` (csrc/host/packing.cc) and fall back to the
pure-Python implementations `*_py` below, which define the semantics and are what the tests compare the
native code against. Output arrays can be allocated in pinned host memory (`pinned=True`) so a packed
chunk goes to the GPU with one async copy per field.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Mapping, Optional, Sequence

import numpy as np

PER_TOKEN_FIELDS = ("old_per_token_logps", "ref_per_token_logps", "sampler_is_weights", "values", "returns")
UNSET_ROUTED_EXPERT = -1


def align_up(offset: int, boundary: int) -> int:
    if boundary <= 0:
        raise ValueError(f"segment_alignment_boundary must be positive, got {boundary}")
    return -(-offset // boundary) * boundary


def _as1d(arr, dtype, name):
    if not isinstance(arr, np.ndarray) or arr.ndim != 1:
        raise ValueError(f"PackItem.{name} must be a 1D numpy array, got {type(arr).__name__} with shape "
                         f"{getattr(arr, 'shape', None)}. Unpad and flatten before packing.")
    return np.ascontiguousarray(arr, dtype=dtype)


@dataclasses.dataclass(frozen=True, kw_only=True)
class PackItem:
    prompt_ids: np.ndarray
    completion_ids: np.ndarray
    completion_mask: np.ndarray
    advantages: np.ndarray
    per_token: Mapping[str, np.ndarray] = dataclasses.field(default_factory=dict)
    policy_version: Optional[np.ndarray] = None
    routed_experts: Optional[np.ndarray] = None   # [p+c-1 or p+c, num_layers, top_k] int16

    def __post_init__(self):
        for name, dt in (("prompt_ids", np.int32), ("completion_ids", np.int32), ("completion_mask", np.float32),
                         ("advantages", np.float32)):
            object.__setattr__(self, name, _as1d(getattr(self, name), dt, name))
        c = self.completion_ids.shape[0]
        for name in ("completion_mask", "advantages"):
            if getattr(self, name).shape[0] != c:
                raise ValueError(f"PackItem.{name} must have length matching completion_ids length; got "
                                 f"{getattr(self, name).shape[0]}, expected {c}.")
        pt = {}
        for key, arr in self.per_token.items():
            if key not in PER_TOKEN_FIELDS:
                raise ValueError(f"Unknown per-token field {key!r}; expected one of {PER_TOKEN_FIELDS}.")
            if not isinstance(arr, np.ndarray) or arr.ndim != 1 or arr.shape[0] != c:
                raise ValueError(f"PackItem.per_token[{key!r}] must be a 1D numpy array of shape (c,)")
            pt[key] = np.ascontiguousarray(arr, dtype=np.float32)
        object.__setattr__(self, "per_token", pt)
        if self.routed_experts is not None:
            n = self.prompt_ids.shape[0] + c
            r = self.routed_experts
            if not isinstance(r, np.ndarray) or r.ndim != 3 or r.shape[0] < max(n - 1, 0) or r.shape[0] > n:
                raise ValueError("PackItem.routed_experts must have shape (p + c - 1 or p + c, num_layers, top_k)")
            object.__setattr__(self, "routed_experts", np.ascontiguousarray(r, dtype=np.int16))

    @property
    def num_tokens(self) -> int:
        return int(self.prompt_ids.shape[0] + self.completion_ids.shape[0])


@dataclasses.dataclass(frozen=True, kw_only=True)
class PackedRow:
    ids: np.ndarray
    prompt_mask: np.ndarray
    completion_mask: np.ndarray
    advantages: np.ndarray
    segment_ids: np.ndarray
    segment_positions: np.ndarray
    per_token: Mapping[str, np.ndarray] = dataclasses.field(default_factory=dict)
    policy_version: Optional[np.ndarray] = None
    num_real_segments: int = 0
    routed_experts: Optional[np.ndarray] = None


@dataclasses.dataclass(frozen=True, kw_only=True)
class PackedChunk:
    ids: np.ndarray
    prompt_mask: np.ndarray
    completion_mask: np.ndarray
    advantages: np.ndarray
    segment_ids: np.ndarray
    segment_positions: np.ndarray
    per_token: Mapping[str, np.ndarray] = dataclasses.field(default_factory=dict)
    policy_versions: tuple = ()
    num_real_segments: tuple = ()
    routed_experts: Optional[np.ndarray] = None
    bin_indices: tuple = ()

    def __len__(self) -> int:
        return int(self.ids.shape[0])

    def __getitem__(self, index):
        if isinstance(index, slice):
            return [self[i] for i in range(*index.indices(len(self)))]
        if index < 0:
            index += len(self)
        if index < 0 or index >= len(self):
            raise IndexError(f"PackedChunk index {index} out of range.")
        return PackedRow(
            ids=self.ids[index], prompt_mask=self.prompt_mask[index], completion_mask=self.completion_mask[index],
            advantages=self.advantages[index], segment_ids=self.segment_ids[index],
            segment_positions=self.segment_positions[index],
            per_token={k: v[index] for k, v in self.per_token.items()},
            policy_version=self.policy_versions[index] if index < len(self.policy_versions) else None,
            num_real_segments=self.num_real_segments[index] if index < len(self.num_real_segments) else 0,
            routed_experts=None if self.routed_experts is None else self.routed_experts[index])

    def __iter__(self):
        return (self[i] for i in range(len(self)))


def carried_per_token_fields(items: Sequence[PackItem]) -> tuple:
    if not items:
        return ()
    return tuple(n for n in PER_TOKEN_FIELDS if all(n in it.per_token for it in items))


# ------------------------------------------------------------------ Python twins
def fill_one_chunk_py(items: Sequence[PackItem], pack_size: int, budget: int, max_segments: int,
                      boundary: int = 1, order: Optional[list] = None):
    """FFD: returns (bins: list[list[idx]], starts: dict idx->offset, leftover: list[idx] ascending)."""
    if boundary <= 0:
        raise ValueError("segment_alignment_boundary must be positive")
    n = len(items)
    if order is None:
        order = sorted(range(n), key=lambda i: -items[i].num_tokens)  # stable
    bins = [[] for _ in range(max(pack_size, 0))]
    starts: dict = {}
    if n == 0 or pack_size <= 0 or max_segments <= 0:
        return bins, starts, sorted(order)
    rem = [budget] * pack_size
    nxt = [0] * pack_size
    segs = [0] * pack_size
    leftover, closed_all = [], False
    for pos, it in enumerate(order):
        if closed_all:
            leftover.append(it)
            continue
        ln = items[it].num_tokens
        placed = False
        if ln <= max(rem):
            for b in range(pack_size):
                if rem[b] >= ln:
                    bins[b].append(it)
                    starts[it] = nxt[b]
                    end = nxt[b] + ln
                    segs[b] += 1
                    if segs[b] >= max_segments:
                        rem[b] = -1
                    else:
                        nxt[b] = align_up(end, boundary)
                        rem[b] = budget - nxt[b]
                    placed = True
                    break
        if not placed:
            leftover.append(it)
            if max(rem) < 0:
                closed_all = True
    return bins, starts, sorted(leftover)


def pack_chunk_py(items: Sequence[PackItem], bins, starts, budget: int, pad_id: int) -> PackedChunk:
    n_bins = len(bins)
    fields = carried_per_token_fields([items[i] for b in bins for i in b])
    any_routed = any(items[i].routed_experts is not None for b in bins for i in b)
    ids = np.full((n_bins, budget), pad_id, np.int32)
    pm = np.zeros((n_bins, budget), np.float32)
    cm = np.zeros((n_bins, budget), np.float32)
    adv = np.zeros((n_bins, budget), np.float32)
    seg = np.zeros((n_bins, budget), np.int32)
    pos = np.zeros((n_bins, budget), np.int32)
    pt = {f: np.zeros((n_bins, budget), np.float32) for f in fields}
    routed = None
    if any_routed:
        shape = next(items[i].routed_experts.shape[1:] for b in bins for i in b if items[i].routed_experts is not None)
        routed = np.full((n_bins, budget) + tuple(shape), UNSET_ROUTED_EXPERT, np.int16)
    nseg = []
    for b, members in enumerate(bins):
        s = 0
        for it in sorted(members, key=lambda i: starts[i]):
            item = items[it]
            p, c = item.prompt_ids.shape[0], item.completion_ids.shape[0]
            o = starts[it]
            if o + p + c > budget:
                raise ValueError("packed row overflows the token budget")
            s += 1
            ids[b, o:o + p] = item.prompt_ids
            ids[b, o + p:o + p + c] = item.completion_ids
            pm[b, o:o + p] = 1
            cm[b, o + p:o + p + c] = item.completion_mask
            adv[b, o + p:o + p + c] = item.advantages
            seg[b, o:o + p + c] = s
            pos[b, o:o + p + c] = np.arange(p + c)
            for f in fields:
                pt[f][b, o + p:o + p + c] = item.per_token[f]
            if routed is not None and item.routed_experts is not None:
                m = min(item.routed_experts.shape[0], p + c)
                routed[b, o:o + m] = item.routed_experts[:m]
        nseg.append(s)
    return PackedChunk(ids=ids, prompt_mask=pm, completion_mask=cm, advantages=adv, segment_ids=seg,
                       segment_positions=pos, per_token=pt, num_real_segments=tuple(nseg), routed_experts=routed,
                       policy_versions=tuple(_row_policy_version(items, m) for m in bins),
                       bin_indices=tuple(tuple(m) for m in bins))


def _row_policy_version(items, members):
    vs = [items[i].policy_version for i in members if items[i].policy_version is not None]
    return np.concatenate([np.atleast_1d(v) for v in vs]) if vs else None


# ------------------------------------------------------------------ native path
def _host():
    try:
        from .. import _lib
        lib = _lib.host()
        lib.tb_pack_ffd.restype = ctypes.c_int
        return lib
    except Exception:
        return None


def _csr(arrays, dtype):
    off = np.zeros(len(arrays) + 1, np.int64)
    np.cumsum([a.shape[0] for a in arrays], out=off[1:])
    flat = np.concatenate(arrays).astype(dtype, copy=False) if arrays and off[-1] > 0 else np.zeros(0, dtype)
    return np.ascontiguousarray(flat), off


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _alloc(shape, dtype, pinned: bool):
    if pinned:
        try:
            import torch
            tdt = {np.int32: torch.int32, np.float32: torch.float32, np.int16: torch.int16}[dtype]
            return torch.empty(shape, dtype=tdt).pin_memory().numpy()
        except Exception:
            pass
    return np.empty(shape, dtype)


def fill_one_chunk(items: Sequence[PackItem], pack_size: int, budget: int, max_segments: int, boundary: int = 1):
    """FFD bin assignment (native when available). Returns (bins, starts, leftover)."""
    lib = _host()
    if lib is None:
        return fill_one_chunk_py(items, pack_size, budget, max_segments, boundary)
    if boundary <= 0:
        raise ValueError("segment_alignment_boundary must be positive")
    n = len(items)
    lengths = np.asarray([it.num_tokens for it in items], np.int32)
    bin_of = np.empty(n, np.int32)
    start_of = np.empty(n, np.int32)
    rc = lib.tb_pack_ffd(_p(lengths), n, int(pack_size), ctypes.c_int64(budget), int(max_segments),
                         ctypes.c_int64(boundary), _p(bin_of), _p(start_of))
    if rc < 0:
        raise ValueError("invalid packing arguments")
    bins = [[] for _ in range(max(pack_size, 0))]
    starts = {}
    placed = [i for i in range(n) if bin_of[i] >= 0]
    for i in sorted(placed, key=lambda i: (bin_of[i], start_of[i])):
        bins[bin_of[i]].append(i)
        starts[i] = int(start_of[i])
    leftover = [i for i in range(n) if bin_of[i] < 0]
    return bins, starts, leftover


def pack_chunk(items: Sequence[PackItem], bins, starts, budget: int, pad_id: int, pinned: bool = False) -> PackedChunk:
    """Row fill (native when available)."""
    lib = _host()
    if lib is None:
        return pack_chunk_py(items, bins, starts, budget, pad_id)
    n = len(items)
    n_bins = len(bins)
    members = [i for b in bins for i in b]
    fields = carried_per_token_fields([items[i] for i in members])
    any_routed = any(items[i].routed_experts is not None for i in members)
    bin_of = np.full(n, -1, np.int32)
    start_of = np.zeros(n, np.int32)
    for b, ms in enumerate(bins):
        for i in ms:
            bin_of[i] = b
            start_of[i] = starts[i]
    pids, poff = _csr([it.prompt_ids for it in items], np.int32)
    cids, coff = _csr([it.completion_ids for it in items], np.int32)
    cmask, _ = _csr([it.completion_mask for it in items], np.float32)
    advs, _ = _csr([it.advantages for it in items], np.float32)
    pts = [_csr([it.per_token.get(f, np.zeros(it.completion_ids.shape[0], np.float32)) for it in items], np.float32)[0]
           for f in fields]
    rl = rk = 0
    routed_flat = roff = None
    if any_routed:
        shape = next(items[i].routed_experts.shape[1:] for i in members if items[i].routed_experts is not None)
        rl, rk = int(shape[0]), int(shape[1])
        rs = [it.routed_experts.reshape(it.routed_experts.shape[0], -1) if it.routed_experts is not None
              else np.zeros((0, rl * rk), np.int16) for it in items]
        roff = np.zeros(n + 1, np.int64)
        np.cumsum([r.shape[0] for r in rs], out=roff[1:])
        routed_flat = np.ascontiguousarray(np.concatenate(rs, axis=0).astype(np.int16))
    out = {k: _alloc((n_bins, budget), dt, pinned) for k, dt in
           (("ids", np.int32), ("pm", np.float32), ("cm", np.float32), ("adv", np.float32), ("seg", np.int32),
            ("pos", np.int32))}
    out_fields = [_alloc((n_bins, budget), np.float32, pinned) for _ in fields]
    out_routed = _alloc((n_bins, budget, rl, rk), np.int16, pinned) if any_routed else None
    nseg = np.zeros(n_bins, np.int32)
    idx = np.asarray(members, np.int32)
    pt_ptrs = (ctypes.c_void_p * max(len(fields), 1))(*[a.ctypes.data for a in pts])
    of_ptrs = (ctypes.c_void_p * max(len(fields), 1))(*[a.ctypes.data for a in out_fields])
    rc = lib.tb_pack_fill(_p(idx), len(members), _p(bin_of), _p(start_of), _p(pids), _p(poff), _p(cids), _p(cmask),
                          _p(advs), _p(coff), pt_ptrs, len(fields), _p(routed_flat), _p(roff), rl, rk, n_bins,
                          ctypes.c_int64(budget), int(pad_id), _p(out["ids"]), _p(out["pm"]), _p(out["cm"]),
                          _p(out["adv"]), _p(out["seg"]), _p(out["pos"]), of_ptrs, _p(out_routed), _p(nseg))
    if rc != 0:
        raise ValueError("packed row overflows the token budget")
    return PackedChunk(ids=out["ids"], prompt_mask=out["pm"], completion_mask=out["cm"], advantages=out["adv"],
                       segment_ids=out["seg"], segment_positions=out["pos"],
                       per_token=dict(zip(fields, out_fields)), num_real_segments=tuple(int(x) for x in nseg),
                       routed_experts=out_routed,
                       policy_versions=tuple(_row_policy_version(items, m) for m in bins),
                       bin_indices=tuple(tuple(m) for m in bins))


def pack_core(items: Sequence[PackItem], pack_size: int, budget: int, pad_id: int, max_segments: Optional[int] = None,
              boundary: int = 1, min_buffered_tokens: int = 0, pinned: bool = False):
    """Pack everything into chunks of `pack_size` rows. Returns (chunks, leftover indices ascending)."""
    max_segments = budget if max_segments is None else max_segments
    remaining = list(range(len(items)))
    chunks = []
    while remaining:
        tokens_left = sum(items[i].num_tokens for i in remaining)
        if min_buffered_tokens > 0 and tokens_left < min_buffered_tokens:
            break
        sub = [items[i] for i in remaining]
        bins, starts, leftover = fill_one_chunk(sub, pack_size, budget, max_segments, boundary)
        if len(leftover) == len(sub):
            raise ValueError("an item is longer than the packing budget and can never be placed")
        bins = [b for b in bins if b]
        chunk = pack_chunk(sub, bins, starts, budget, pad_id, pinned)
        mapped = tuple(tuple(remaining[i] for i in b) for b in bins)
        chunks.append(dataclasses.replace(chunk, bin_indices=mapped))
        remaining = [remaining[i] for i in leftover]
    return chunks, sorted(remaining)


def count_router_replay_forced_tokens(routed: np.ndarray, segment_ids: np.ndarray) -> tuple:
    """(real tokens, tokens whose layer-0 expert list is fully valid and duplicate-free)."""
    routed = np.ascontiguousarray(routed, np.int16)
    segment_ids = np.ascontiguousarray(segment_ids, np.int32)
    B, T, L, k = routed.shape
    lib = _host()
    if lib is not None:
        out = np.zeros(2, np.int64)
        lib.tb_count_router_replay_forced(_p(routed), _p(segment_ids), ctypes.c_int64(B), ctypes.c_int64(T), L, k, _p(out))
        return int(out[0]), int(out[1])
    real = segment_ids > 0
    l0 = routed[:, :, 0, :]
    valid = (l0 >= 0).all(-1)
    srt = np.sort(l0, axis=-1)
    nodup = (np.diff(srt, axis=-1) != 0).all(-1) if k > 1 else np.ones_like(valid)
    return int(real.sum()), int((real & valid & nodup).sum())
