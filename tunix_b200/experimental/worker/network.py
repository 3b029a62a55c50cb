"""Bulk data plane beside the gRPC control plane (tunix/experimental/worker/network.py: striped TCP for payloads of
512 KiB and more, chunk serialisation that does not hold the interpreter lock).

Weights are the one thing in an RL job that is large: pickling a few GB into gRPC messages copies every byte several
times under the GIL. Here arrays never enter a pickle:

  * `split_arrays(obj)` takes the numpy arrays out of a nested payload and leaves small `ArrayRef` markers behind;
    `ArrayBundle` lays the arrays end to end (64-byte aligned) behind a JSON table of dtype / shape / offset.
  * `send_bulk` cuts the bundle into `stripes` contiguous ranges and sends each over its own TCP connection with
    `socket.sendall(memoryview)`; `BulkReceiver` reads every stripe with `recv_into` straight into its slice of ONE
    preallocated buffer. Socket calls release the GIL, so the stripes really move side by side, and the receiver's
    arrays are `np.frombuffer` views of that buffer: one copy on the way in (into the bundle), none on the way out.
  * the small remainder (the skeleton with the markers, and a `BulkHandle` naming the transfer) goes through the
    ordinary RPC; `join_arrays` puts the views back in place on the other side.

Every connection starts with a fixed header (magic, token digest, transfer id, total size, offset, length); a
receiver with a token drops connections whose digest does not match. Transfers that never complete are dropped
after `ttl_s`."""
from __future__ import annotations

import hashlib
import hmac
import json
import os
import socket
import struct
import threading
import time
from typing import Any, Optional

import numpy as np

BULK_THRESHOLD = 512 << 10
_MAGIC = b"TB2B"
_HDR = struct.Struct("!4s32s16sQQQ")                        # magic, token digest, transfer id, total, offset, length
_ALIGN = 64


def _digest(token: Optional[str]) -> bytes:
    return hashlib.sha256((token or "").encode()).digest()


class ArrayRef:
    __slots__ = ("index",)

    def __init__(self, index: int):
        self.index = index

    def __reduce__(self):
        return (ArrayRef, (self.index,))


class BulkHandle:
    """Names a finished or pending transfer on the receiving side."""
    __slots__ = ("transfer_id", "nbytes")

    def __init__(self, transfer_id: bytes, nbytes: int):
        self.transfer_id, self.nbytes = transfer_id, nbytes

    def __reduce__(self):
        return (BulkHandle, (self.transfer_id, self.nbytes))


def split_arrays(obj: Any, min_bytes: int = 0):
    """(skeleton, arrays): numpy arrays of at least `min_bytes` are replaced by `ArrayRef`s, depth first."""
    arrays: list = []

    def walk(o):
        if isinstance(o, np.ndarray) and o.nbytes >= min_bytes and o.dtype != object:
            arrays.append(o)
            return ArrayRef(len(arrays) - 1)
        if isinstance(o, dict):
            return {k: walk(v) for k, v in o.items()}
        if isinstance(o, tuple):
            return tuple(walk(v) for v in o)
        if isinstance(o, list):
            return [walk(v) for v in o]
        return o
    return walk(obj), arrays


def join_arrays(skeleton: Any, arrays: list):
    def walk(o):
        if isinstance(o, ArrayRef):
            return arrays[o.index]
        if isinstance(o, dict):
            return {k: walk(v) for k, v in o.items()}
        if isinstance(o, tuple):
            return tuple(walk(v) for v in o)
        if isinstance(o, list):
            return [walk(v) for v in o]
        return o
    return walk(skeleton)


class ArrayBundle:
    """[u64 table length][JSON table][padding][array 0][padding][array 1]..."""

    @staticmethod
    def pack(arrays: list, out: Optional[bytearray] = None) -> bytearray:
        """`out`: a buffer of an earlier pack to fill again when the size still fits (its pages are already mapped)."""
        table, off = [], 0
        for a in arrays:
            off = -(-off // _ALIGN) * _ALIGN
            table.append({"dtype": a.dtype.str, "shape": list(a.shape), "offset": off, "nbytes": int(a.nbytes)})
            off += a.nbytes
        head = json.dumps(table).encode()
        base = -(-(8 + len(head)) // _ALIGN) * _ALIGN
        buf = out if out is not None and len(out) == base + off else bytearray(base + off)
        struct.pack_into("!Q", buf, 0, len(head))
        buf[8:8 + len(head)] = head
        mv = memoryview(buf)
        for a, t in zip(arrays, table):
            if a.nbytes:
                dst = np.frombuffer(mv[base + t["offset"]: base + t["offset"] + a.nbytes], dtype=a.dtype).reshape(a.shape)
                np.copyto(dst, a)                           # one pass, releases the GIL for large arrays
        return buf

    @staticmethod
    def unpack(buf) -> list:
        mv = memoryview(buf)
        (n,) = struct.unpack_from("!Q", mv, 0)
        table = json.loads(bytes(mv[8:8 + n]))
        base = -(-(8 + n) // _ALIGN) * _ALIGN
        out = []
        for t in table:
            a = np.frombuffer(mv[base + t["offset"]: base + t["offset"] + t["nbytes"]], dtype=np.dtype(t["dtype"]))
            out.append(a.reshape(t["shape"]))
        return out


def _recv_exact(sock: socket.socket, view: memoryview) -> bool:
    got = 0
    while got < len(view):
        n = sock.recv_into(view[got:], len(view) - got)
        if n == 0:
            return False
        got += n
    return True


class BulkReceiver:
    def __init__(self, host: str = "127.0.0.1", port: int = 0, token: Optional[str] = None, ttl_s: float = 600.0,
                 max_transfer_bytes: int = 64 << 30):
        self._digest, self.ttl_s, self.max_transfer_bytes = _digest(token), ttl_s, max_transfer_bytes
        self._sock = socket.create_server((host, port), backlog=64)
        self.host, self.port = host, self._sock.getsockname()[1]
        self._lock = threading.Lock()
        self._cv = threading.Condition(self._lock)
        self._transfers: dict = {}                          # id -> [buffer, bytes remaining, created]
        self._closed = False
        self._pool: dict = {}                               # size -> buffers handed back with release()
        self.pool_limit = 2
        self.bytes_received = self.buffers_reused = 0
        self._thread = threading.Thread(target=self._accept, name="tunix-b200-bulk-accept", daemon=True)
        self._thread.start()

    @property
    def address(self) -> str:
        return f"{self.host}:{self.port}"

    def _accept(self) -> None:
        while not self._closed:
            try:
                conn, _ = self._sock.accept()
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), name="tunix-b200-bulk-stripe", daemon=True).start()

    def _serve(self, conn: socket.socket) -> None:
        with conn:
            conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            head = bytearray(_HDR.size)
            if not _recv_exact(conn, memoryview(head)):
                return
            magic, digest, tid, total, offset, length = _HDR.unpack(head)
            if magic != _MAGIC or not hmac.compare_digest(digest, self._digest):
                return
            if total > self.max_transfer_bytes or offset + length > total:
                return
            with self._lock:
                self._expire()
                ent = self._transfers.get(tid)
                if ent is None:
                    spare = self._pool.get(total)
                    if spare:
                        buf = spare.pop()
                        self.buffers_reused += 1
                    else:
                        buf = bytearray(total)
                    ent = self._transfers[tid] = [buf, total, time.monotonic()]
                elif len(ent[0]) != total:
                    return
            ok = _recv_exact(conn, memoryview(ent[0])[offset:offset + length])
            try:
                conn.sendall(b"\x01" if ok else b"\x00")    # the sender learns that its stripe has landed
            except OSError:
                pass
            if ok:
                with self._cv:
                    ent[1] -= length
                    self.bytes_received += length
                    self._cv.notify_all()

    def _expire(self) -> None:
        now = time.monotonic()
        for tid in [t for t, e in self._transfers.items() if now - e[2] > self.ttl_s]:
            del self._transfers[tid]

    def take(self, transfer_id: bytes, timeout: Optional[float] = 60.0) -> bytearray:
        """The completed buffer of a transfer (removed from the receiver); waits for stripes still on their way."""
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cv:
            while True:
                ent = self._transfers.get(transfer_id)
                if ent is not None and ent[1] == 0:
                    del self._transfers[transfer_id]
                    return ent[0]
                left = None if deadline is None else deadline - time.monotonic()
                if left is not None and left <= 0:
                    raise TimeoutError(f"transfer {transfer_id.hex()} is incomplete"
                                       + ("" if ent is None else f" ({ent[1]} bytes missing)"))
                self._cv.wait(left)

    def release(self, buf: bytearray) -> None:
        """Hand a taken buffer back for the next transfer of the same size. First-touch page faults of a fresh
        buffer cost more than the copy itself (measured: a new 512 MiB buffer fills at about 0.5 GB/s, a reused one
        several times faster), and weight payloads have the same size every round. Only for callers that keep no
        view of the buffer."""
        with self._lock:
            spare = self._pool.setdefault(len(buf), [])
            if len(spare) < self.pool_limit:
                spare.append(buf)

    def close(self) -> None:
        self._closed = True
        self._pool.clear()
        try:
            self._sock.close()
        except OSError:
            pass


def send_bulk(address: str, data, *, stripes: int = 4, token: Optional[str] = None, transfer_id: Optional[bytes] = None,
              timeout: Optional[float] = 600.0) -> BulkHandle:
    """Send one buffer as `stripes` parallel TCP streams; returns when every stripe has been acknowledged."""
    mv = memoryview(data).cast("B")
    total = len(mv)
    tid = transfer_id or os.urandom(16)
    host, port = address.rsplit(":", 1)
    n = max(1, min(stripes, -(-total // (256 << 10)) or 1))
    step = -(-total // n) if total else 0
    ranges = [(i * step, min(step, total - i * step)) for i in range(n)] if total else [(0, 0)]
    errors: list = []

    def stripe(offset: int, length: int) -> None:
        try:
            with socket.create_connection((host, int(port)), timeout=timeout) as s:
                s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                s.sendall(_HDR.pack(_MAGIC, _digest(token), tid, total, offset, length))
                if length:
                    s.sendall(mv[offset:offset + length])
                ack = s.recv(1)
                if ack != b"\x01":
                    raise ConnectionError("the receiver dropped the stripe (token or size mismatch)")
        except BaseException as e:
            errors.append(e)
    threads = [threading.Thread(target=stripe, args=r) for r in ranges[1:]]
    for t in threads:
        t.start()
    stripe(*ranges[0])
    for t in threads:
        t.join()
    if errors:
        raise ConnectionError(f"bulk transfer to {address} failed: {errors[0]!r}") from errors[0]
    return BulkHandle(tid, total)
