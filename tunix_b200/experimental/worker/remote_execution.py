"""Workers behind a gRPC endpoint (tunix/experimental/worker/remote_execution.py, network.py, in miniature).

`serve_worker(worker, address)` exposes a worker object's public methods over one generic unary RPC
(`/tunix_b200.Worker/Call`); `RemoteWorker(address)` is the proxy the orchestrator registers instead of the
object itself: `submit`, `sync_weights`, `start`, `stop`, `info`, `state` and any other public method go over the
wire. Payloads are cloudpickle frames (method name, args, kwargs -> ("ok", value) | ("err", exception)), large
ones are split into chunks on a client-streaming RPC (`/tunix_b200.Worker/CallChunked`), so a weight payload does
not have to fit one message. Weight payloads whose numpy arrays add up to 512 KiB or more skip the pickle
altogether: the arrays travel over the striped TCP bulk plane of `network.py` and only a handle and the payload's
skeleton go through the RPC.

Unpickling executes code: the endpoint is meant for the private network of one training job and must not be
reachable from anywhere else. It binds to the loopback interface unless told otherwise. With a shared token every
request frame is `magic | HMAC-SHA256(token, body) | body`; the server checks the tag with a constant-time
comparison BEFORE it unpickles the body and answers UNAUTHENTICATED otherwise, so a peer without the token cannot
make the server load a pickle. Without a token every peer that reaches the port can run code: do that on loopback
only. grpcio and cloudpickle are optional dependencies; importing this module without them raises ImportError."""
from __future__ import annotations

import hashlib
import hmac
import threading
from concurrent import futures
from typing import Any, Iterator, Optional

import cloudpickle
import grpc

from ..common.datatypes import WorkerState

_SERVICE = "tunix_b200.Worker"
_CHUNK = 4 << 20
_MAX_MSG = 64 << 20
_OPTS = [("grpc.max_send_message_length", _MAX_MSG), ("grpc.max_receive_message_length", _MAX_MSG)]
_PRIVATE = ("_",)


class RemoteError(RuntimeError):
    """The remote method raised; `__cause__` is the original exception when it could be pickled."""


def _ident(b: bytes) -> bytes:
    return b


_MAGIC = b"TBW1"
_TAG_LEN = 32


def _seal(body: bytes, token: Optional[str]) -> bytes:
    """Request frame: magic, then the HMAC-SHA256 tag of the body under the shared token (zeros without one)."""
    tag = hmac.new(token.encode(), body, hashlib.sha256).digest() if token else b"\0" * _TAG_LEN
    return _MAGIC + tag + body


def _open(frame: bytes, token: Optional[str]) -> Optional[bytes]:
    """The body of an authentic frame, None otherwise. Nothing of the body is interpreted before the tag matched."""
    head = len(_MAGIC) + _TAG_LEN
    if len(frame) < head or frame[:len(_MAGIC)] != _MAGIC:
        return None
    body = frame[head:]
    if token:
        want = hmac.new(token.encode(), body, hashlib.sha256).digest()
        if not hmac.compare_digest(frame[len(_MAGIC):head], want):
            return None
    return body


class _Servicer:
    def __init__(self, worker, token: Optional[str], bulk=None):
        self.worker, self.token, self.bulk = worker, token, bulk
        self._lock = threading.Lock()

    def _resolve_bulk(self, args, kwargs):
        """Arguments that arrived over the bulk plane: ("__bulk__", handle, skeleton) -> the payload with its arrays."""
        from .network import ArrayBundle, BulkHandle, join_arrays

        taken = []

        def fix(a):
            if isinstance(a, tuple) and len(a) == 3 and a[0] == "__bulk__" and isinstance(a[1], BulkHandle):
                if self.bulk is None:
                    raise RuntimeError("this server has no bulk plane")
                taken.append(self.bulk.take(a[1].transfer_id))
                return join_arrays(a[2], ArrayBundle.unpack(taken[-1]))
            return a
        return tuple(fix(a) for a in args), {k: fix(v) for k, v in kwargs.items()}, taken

    def _dispatch(self, frame: bytes, context=None) -> bytes:
        blob = _open(frame, self.token)
        if blob is None:                                # rejected unread: no byte of it reaches the unpickler
            if context is not None:
                context.abort(grpc.StatusCode.UNAUTHENTICATED, "bad or missing token")
            raise PermissionError("bad or missing token")
        try:
            name, args, kwargs = cloudpickle.loads(blob)
            if name == "__bulk_address__":
                return cloudpickle.dumps(("ok", None if self.bulk is None else self.bulk.address))
            if name.startswith(_PRIVATE):
                raise AttributeError(f"{name!r} is not a remote method")
            args, kwargs, taken = self._resolve_bulk(args, kwargs)
            attr = getattr(self.worker, name)
            value = attr(*args, **kwargs) if callable(attr) else attr
            if taken and getattr(self.worker, "releases_bulk_payloads", False):
                del args, kwargs                            # the worker copied what it needs: the buffers serve the next round
                for buf in taken:
                    self.bulk.release(buf)
            return cloudpickle.dumps(("ok", value))
        except BaseException as e:                      # the failure travels back; the server keeps serving
            try:
                return cloudpickle.dumps(("err", e))
            except Exception:
                return cloudpickle.dumps(("err", RuntimeError(repr(e))))

    def call(self, request: bytes, context) -> bytes:
        return self._dispatch(request, context)

    def call_chunked(self, request_iterator: Iterator[bytes], context) -> bytes:
        return self._dispatch(b"".join(request_iterator), context)


class WorkerServer:
    def __init__(self, worker, address: str = "127.0.0.1:0", token: Optional[str] = None, max_threads: int = 16,
                 bulk: bool = True):
        self.bulk = None
        if bulk:
            from .network import BulkReceiver
            self.bulk = BulkReceiver(address.rsplit(":", 1)[0], 0, token)
        svc = _Servicer(worker, token, self.bulk)
        self._server = grpc.server(futures.ThreadPoolExecutor(max_workers=max_threads), options=_OPTS)
        handlers = {
            "Call": grpc.unary_unary_rpc_method_handler(svc.call, request_deserializer=_ident, response_serializer=_ident),
            "CallChunked": grpc.stream_unary_rpc_method_handler(svc.call_chunked, request_deserializer=_ident,
                                                                response_serializer=_ident),
        }
        self._server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(_SERVICE, handlers),))
        host = address.rsplit(":", 1)[0]
        self.port = self._server.add_insecure_port(address)
        if self.port == 0:
            raise OSError(f"could not bind {address}")
        self.address = f"{host}:{self.port}"
        self._server.start()

    def stop(self, grace: float = 1.0) -> None:
        self._server.stop(grace).wait()
        if self.bulk is not None:
            self.bulk.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()


def serve_worker(worker, address: str = "127.0.0.1:0", token: Optional[str] = None) -> WorkerServer:
    return WorkerServer(worker, address, token)


class RemoteWorker:
    """Client-side stand-in for a worker served by `serve_worker`. Unknown attributes become remote calls."""

    def __init__(self, address: str, token: Optional[str] = None, timeout: Optional[float] = 600.0):
        self.address, self._token, self._timeout = address, token, timeout
        self._channel = grpc.insecure_channel(address, options=_OPTS)
        self._call = self._channel.unary_unary(f"/{_SERVICE}/Call", request_serializer=_ident, response_deserializer=_ident)
        self._call_chunked = self._channel.stream_unary(f"/{_SERVICE}/CallChunked", request_serializer=_ident,
                                                        response_deserializer=_ident)
        self._info = None
        self._bulk_address: Any = False                     # False: not asked yet; None: the server has none
        self.bulk_stripes = 4
        self._pack_buf = None
        self.bulk_bytes_sent = 0

    def _via_bulk(self, payload: Any) -> Any:
        """Large array payloads leave the pickle: arrays over striped TCP, the skeleton over the RPC."""
        from .network import BULK_THRESHOLD, ArrayBundle, send_bulk, split_arrays
        if not isinstance(payload, (dict, list, tuple)):
            return payload
        skeleton, arrays = split_arrays(payload, min_bytes=4096)
        if sum(a.nbytes for a in arrays) < BULK_THRESHOLD:
            return payload
        if self._bulk_address is False:
            self._bulk_address = self._invoke("__bulk_address__")
        if self._bulk_address is None:
            return payload
        host = self.address.rsplit(":", 1)[0]
        target = f"{host}:{self._bulk_address.rsplit(':', 1)[1]}"      # the host we reach it by, the port it listens on
        self._pack_buf = ArrayBundle.pack(arrays, out=self._pack_buf)      # same size every round: the buffer is kept
        handle = send_bulk(target, self._pack_buf, stripes=self.bulk_stripes, token=self._token, timeout=self._timeout)
        self.bulk_bytes_sent += handle.nbytes
        return ("__bulk__", handle, skeleton)

    def _invoke(self, name: str, *args, **kwargs) -> Any:
        blob = _seal(cloudpickle.dumps((name, args, kwargs)), self._token)
        try:
            reply = self._send(blob)
        except grpc.RpcError as e:
            if e.code() == grpc.StatusCode.UNAUTHENTICATED:
                raise RemoteError(f"{name} refused by {self.address}: bad or missing token") from e
            raise
        kind, value = cloudpickle.loads(reply)
        if kind == "err":
            raise RemoteError(f"{name} failed on {self.address}: {value!r}") from (value if isinstance(value, BaseException) else None)
        return value

    def _send(self, blob: bytes) -> bytes:
        if len(blob) > _CHUNK:
            reply = self._call_chunked((blob[i:i + _CHUNK] for i in range(0, len(blob), _CHUNK)), timeout=self._timeout)
        else:
            reply = self._call(blob, timeout=self._timeout)
        return reply

    # the methods the orchestrator and the registry use, spelled out so that they show up in completion and docs
    def info(self):
        if self._info is None:
            self._info = self._invoke("info")
        return self._info

    @property
    def worker_id(self) -> str:
        return self.info().worker_id

    @property
    def state(self) -> WorkerState:
        return self._invoke("state")

    @property
    def policy_version(self) -> int:
        return self._invoke("policy_version")

    def start(self) -> None:
        return self._invoke("start")

    def stop(self) -> None:
        return self._invoke("stop")

    def submit(self, request: Any) -> Any:
        return self._invoke("submit", request)

    def sync_weights(self, version: int, payload: Any = None) -> None:
        return self._invoke("sync_weights", version, self._via_bulk(payload))

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *a, **kw: self._invoke(name, *a, **kw)

    def close(self) -> None:
        self._channel.close()
