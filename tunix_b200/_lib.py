"""ctypes bindings for the in-tree native libraries.

`cuda()` returns the sm_100a kernel library, `host()` the C++ host library. Both are
built on first use when the shared object is missing or stale (`_build.py`). On a
machine with a GPU a missing CUDA library is a hard error: there is no silent
PyTorch fallback for the GPU path.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import _build

_lock = threading.Lock()
_cuda_lib = None
_host_lib = None

P = c_void_p
LL = c_longlong
I = c_int
F = c_float
U = ctypes.c_uint

_CUDA_SIGS = {
    "tb_gemm_bf16": [P, P, P, I, I, I, LL, LL, LL, I, P, P, LL, F, P, I, P],
    "tb_gemm_bf16_ext": [P, P, P, I, I, I, LL, LL, LL, I, P, P, LL, F, P, P, I, LL, LL, P, P],
    "tb_tmap_cache_clear": [],
    "tb_rmsnorm_fwd": [P, LL, P, P, LL, P, I, I, F, F, P],
    "tb_rmsnorm_bwd": [P, LL, P, LL, P, P, P, LL, P, I, I, F, I, P],
    "tb_rope": [P, LL, P, P, P, LL, I, I, I, P],
    "tb_glu_fwd": [P, LL, P, LL, P, LL, LL, I, I, P],
    "tb_glu_bwd": [P, LL, P, LL, P, LL, P, LL, P, LL, LL, I, I, P],
    "tb_embedding_fwd": [P, P, LL, P, LL, LL, I, I, F, P],
    "tb_embedding_bwd": [P, P, LL, P, LL, LL, I, I, F, P],
    "tb_add_bf16": [P, P, P, LL, P],
    "tb_logsoftmax_gather": [P, LL, P, P, P, P, I, I, F, F, P],
    "tb_dlogits": [P, LL, P, P, P, P, P, P, LL, I, I, F, F, P],
    "tb_sumsq": [P, LL, I, P, P],
    "tb_adamw": [P, P, P, P, I, P, LL, F, F, F, F, F, F, F, F, F, P, P, P],
    "tb_sgd": [P, P, P, I, P, LL, F, F, F, F, P],
    "tb_cast_f32_bf16": [P, P, LL, F, P],
    "tb_cast_bf16_f32": [P, P, LL, F, I, P],
}


def _bind(lib, sigs):
    for name, argtypes in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int


def register_cuda_sigs(sigs: dict) -> None:
    """Let op modules declare the signatures of the entry points they call."""
    _CUDA_SIGS.update(sigs)
    if _cuda_lib is not None:
        _bind(_cuda_lib, sigs)


def cuda():
    global _cuda_lib
    if _cuda_lib is None:
        with _lock:
            if _cuda_lib is None:
                path = _build.build_cuda()
                lib = ctypes.CDLL(str(path))
                _bind(lib, _CUDA_SIGS)
                _cuda_lib = lib
    return _cuda_lib


def host():
    global _host_lib
    if _host_lib is None:
        with _lock:
            if _host_lib is None:
                import os
                path = os.environ.get("TUNIX_B200_HOST_LIB") or _build.build_host()      # override: a sanitizer build
                _host_lib = ctypes.CDLL(str(path))
    return _host_lib


def has_gpu() -> bool:
    return torch.cuda.is_available()


_home_device = None


def stream_ptr() -> int:
    """Stream of the calling thread on this process's GPU. One process drives one GPU; a helper thread (rollout
    producer, agentic loop, engine group) starts with CUDA device 0 current, so its launches would go to the
    wrong GPU on every rank but the first: such a thread is moved to the process's device on its first launch."""
    global _home_device
    cur = torch.cuda.current_device()
    if _home_device is None:
        if threading.current_thread() is threading.main_thread():
            _home_device = cur
    elif cur != _home_device and threading.current_thread() is not threading.main_thread():
        torch.cuda.set_device(_home_device)
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


_status_bufs: dict = {}


def status_buffer(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits write their error code to."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    if dev.type != "cuda":
        raise ValueError("status buffers live on CUDA devices")
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    buf = _status_bufs.get(idx)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _status_bufs[idx] = buf
    return buf


def raise_if_kernel_error(device=None) -> None:
    """Synchronising check of the status word; raises if any bounded wait gave up."""
    buf = status_buffer(device)
    code = int(buf[0].item())
    if code != 0:
        buf.zero_()
        names = {1: "TMA producer wait", 2: "MMA wait", 3: "epilogue wait", 4: "flag wait", 5: "bad argument"}
        raise RuntimeError(f"tunix_b200 kernel reported status {code} ({names.get(code, 'unknown')}): a bounded wait timed out")
