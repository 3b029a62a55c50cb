"""Reader for checkpoints that Orbax wrote in its OCDBT layout (the layout of the reference's committed fixture,
tests/sft/test_data/checkpoints/1/model_params, and the default of `orbax.checkpoint` since 0.5).

An OCDBT directory is a key-value store packed into a few files (TensorStore's "optionally-cooperative distributed
B+tree"): `manifest.ocdbt` names the root B+tree node of the latest version; nodes live in `d/<id>` files; leaf
entries map keys such as `layers.0.weight/.zarray` and `layers.0.weight/0.1` to values that are either stored in the
node itself or referenced as (file, offset, length). On top of that store sit ordinary zarr-v2 arrays: `.zarray`
JSON plus one (optionally zstd-compressed) chunk per grid cell. This module walks the tree and assembles the
arrays; nothing is written.

Every OCDBT file is: 4-byte magic, uint64 total length, varint format version (0), one byte compression (0 none,
1 zstd), body, CRC-32C. Bodies as decoded here:

  manifest   uuid[16] | manifest kind | max inline value bytes | max decoded node bytes | arity log2 (u8) |
             compression (varint; zstd is followed by an int32 level) | data file table | inline version entries
             (column by column: generation, root height u8, file id, offset, length, key count, tree bytes,
             indirect bytes, commit time u64) | version-tree node references
  B+tree node  height (u8) | data file table | entry count | key prefix lengths (entries 1..n-1) | key suffix
             lengths | [interior: common-prefix lengths] | key suffix bytes |
             leaf: value lengths | value kinds (u8: 0 inline, 1 referenced) | file ids and offsets of the referenced
                   values | inline value bytes
             interior: child file ids | offsets | lengths | key counts | tree bytes | indirect bytes
  data file table  count | path prefix lengths (1..n-1) | suffix lengths | base-path lengths | suffix bytes

The leaf / inline-value path is verified against the reference's fixture; interior nodes and referenced values
follow the same published format description but no checkpoint large enough to contain them is available offline.
zstd decoding uses `pyarrow` (the only zstd binding in this environment).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Optional

import numpy as np

MAGIC_MANIFEST, MAGIC_BTREE = 0x0CDB3A2A, 0x0CDB20DE


def _zstd(buf: bytes) -> bytes:
    """Decompress one zstd frame (streaming, so frames that do not record their content size work too: zarr chunks
    written by TensorStore do not)."""
    if buf[:4] != b"\x28\xb5\x2f\xfd":
        raise ValueError("not a zstd frame")
    try:
        import pyarrow as pa
    except ImportError as e:       # pragma: no cover
        raise ImportError("reading zstd-compressed OCDBT checkpoints needs pyarrow") from e
    with pa.CompressedInputStream(pa.BufferReader(buf), "zstd") as f:
        return f.read()


class _Reader:
    def __init__(self, data: bytes):
        self.d, self.p = data, 0

    def u8(self) -> int:
        v = self.d[self.p]
        self.p += 1
        return v

    def varint(self) -> int:
        shift = out = 0
        while True:
            b = self.d[self.p]
            self.p += 1
            out |= (b & 0x7F) << shift
            if not b & 0x80:
                return out
            shift += 7

    def varints(self, n: int) -> list:
        return [self.varint() for _ in range(n)]

    def take(self, n: int) -> bytes:
        v = self.d[self.p:self.p + n]
        if len(v) != n:
            raise ValueError("truncated OCDBT record")
        self.p += n
        return v


def _file_body(raw: bytes, want_magic: int) -> _Reader:
    magic, length = struct.unpack(">I", raw[:4])[0], struct.unpack("<Q", raw[4:12])[0]
    if magic != want_magic:
        raise ValueError(f"OCDBT magic {magic:#x}, expected {want_magic:#x}")
    if length != len(raw):
        raise ValueError(f"OCDBT record says {length} bytes, file slice has {len(raw)}")
    r = _Reader(raw[12:-4])
    if r.varint() != 0:
        raise ValueError("unknown OCDBT format version")
    comp = r.u8()
    rest = r.d[r.p:]
    return _Reader(_zstd(rest) if comp == 1 else rest)


def _data_file_table(r: _Reader) -> list:
    n = r.varint()
    prefix = [0] + r.varints(max(n - 1, 0))
    suffix = r.varints(n)
    r.varints(n)                                  # base-path lengths: which part of the path is the directory
    paths, prev = [], b""
    for i in range(n):
        prev = prev[:prefix[i]] + r.take(suffix[i])
        paths.append(prev.decode())
    return paths


class OcdbtStore:
    """Read-only view of one OCDBT directory as {key: bytes}."""

    def __init__(self, directory: str):
        self.dir = directory
        with open(os.path.join(directory, "manifest.ocdbt"), "rb") as f:
            r = _file_body(f.read(), MAGIC_MANIFEST)
        r.take(16)                                # uuid
        r.varint()                                # manifest kind
        r.varint()                                # max inline value bytes
        r.varint()                                # max decoded node bytes
        r.u8()                                    # version tree arity log2
        if r.varint() == 1:
            r.take(4)                             # zstd level
        files = _data_file_table(r)
        n = r.varint()
        if n == 0:
            raise ValueError("OCDBT manifest holds no version")
        gen = r.varints(n)
        height = [r.u8() for _ in range(n)]
        fid, off, ln = r.varints(n), r.varints(n), r.varints(n)
        latest = max(range(n), key=lambda i: gen[i])
        self._root = (height[latest], files[fid[latest]] if ln[latest] else None, off[latest], ln[latest])
        self._cache: Optional[dict] = None

    def _read(self, path: str, offset: int, length: int) -> bytes:
        with open(os.path.join(self.dir, path), "rb") as f:
            f.seek(offset)
            return f.read(length)

    def _walk(self, path: str, offset: int, length: int, prefix: bytes, out: dict) -> None:
        r = _file_body(self._read(path, offset, length), MAGIC_BTREE)
        height = r.u8()
        files = _data_file_table(r)
        n = r.varint()
        kpre = [0] + r.varints(max(n - 1, 0))
        ksuf = r.varints(n)
        common = r.varints(n) if height > 0 else None
        keys, prev = [], b""
        for i in range(n):
            prev = prev[:kpre[i]] + r.take(ksuf[i])
            keys.append(prev)
        if height == 0:
            vlen = r.varints(n)
            kind = [r.u8() for _ in range(n)]
            ref = [i for i in range(n) if kind[i] == 1]
            rfile = dict(zip(ref, r.varints(len(ref))))
            roff = dict(zip(ref, r.varints(len(ref))))
            for i in range(n):
                if kind[i] == 0:
                    out[prefix + keys[i]] = r.take(vlen[i])
                else:
                    out[prefix + keys[i]] = self._read(files[rfile[i]], roff[i], vlen[i])
            return
        cfile, coff, clen = r.varints(n), r.varints(n), r.varints(n)
        for i in range(n):
            # a child's keys are relative to the part of its separator key that the subtree shares
            self._walk(files[cfile[i]], coff[i], clen[i], prefix + keys[i][:common[i]], out)

    def items(self) -> dict:
        if self._cache is None:
            out: dict = {}
            _, path, off, ln = self._root
            if path is not None:
                self._walk(path, off, ln, b"", out)
            self._cache = {k.decode(): v for k, v in out.items()}
        return self._cache


def _decode_chunk(raw: bytes, compressor) -> bytes:
    if compressor is None:
        return raw
    if compressor.get("id") == "zstd":
        return _zstd(raw)
    raise ValueError(f"zarr compressor {compressor.get('id')!r} is not supported")


def read_zarr_array(store: dict, name: str) -> np.ndarray:
    """Assemble the zarr-v2 array stored under `name/` in a {key: bytes} store."""
    meta = json.loads(store[f"{name}/.zarray"])
    shape, chunks = tuple(meta["shape"]), tuple(meta["chunks"])
    sep = meta.get("dimension_separator", ".")
    dt = meta["dtype"]
    np_dt = np.dtype("<u2") if dt == "bfloat16" else np.dtype(dt)
    out = np.zeros(shape, dtype=np_dt)
    if meta.get("fill_value") not in (None, 0, 0.0) and dt != "bfloat16":
        out[...] = meta["fill_value"]
    grid = [range(-(-s // c)) for s, c in zip(shape, chunks)] or [range(1)]
    for idx in np.ndindex(*[len(g) for g in grid]):
        key = f"{name}/" + (sep.join(str(i) for i in idx) if shape else "0")
        raw = store.get(key)
        if raw is None:
            continue                               # an absent chunk holds the fill value
        block = np.frombuffer(_decode_chunk(raw, meta.get("compressor")), dtype=np_dt).reshape(chunks or (1,), order=meta.get("order", "C"))
        sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, shape))
        out[sl] = block[tuple(slice(0, s.stop - s.start) for s in sl)] if shape else block.reshape(())
    return out


def load_tree(directory: str) -> dict:
    """{('w1', 'kernel', 'value'): array} for every array of an Orbax OCDBT item directory; the key tuples come from
    its `_METADATA` when present, else from splitting the array names at the dots. bfloat16 arrays come back as
    uint16 bit patterns (numpy has no bfloat16); `to_torch` turns them into torch.bfloat16."""
    store = OcdbtStore(directory).items()
    names = sorted({k.rsplit("/", 1)[0] for k in store if k.endswith("/.zarray")})
    keys = {}
    md_path = os.path.join(directory, "_METADATA")
    if os.path.exists(md_path):
        with open(md_path) as f:
            for info in json.load(f).get("tree_metadata", {}).values():
                tup = tuple(k["key"] for k in info["key_metadata"])
                keys[".".join(tup)] = tup
    return {keys.get(n, tuple(n.split("."))): read_zarr_array(store, n) for n in names}


def to_torch(array: np.ndarray, dtype_name: Optional[str] = None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(array))
    return t.view(torch.bfloat16) if dtype_name == "bfloat16" else t
