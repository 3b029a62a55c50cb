"""Launcher for the fused sampling kernel (csrc/sampling.cu)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib
from . import kernels as K

_lib.register_cuda_sigs({
    "tb_sample": [_lib.P, _lib.LL, _lib.I, _lib.I, _lib.F, _lib.I, _lib.F, ctypes.c_ulonglong, _lib.I, _lib.P, _lib.P,
                  _lib.P, _lib.P],
    "tb_sample_ex": [_lib.P, _lib.LL, _lib.I, _lib.I, _lib.F, _lib.I, _lib.F, ctypes.c_ulonglong, _lib.I, _lib.P, _lib.P,
                     _lib.P, _lib.F, _lib.P, _lib.I, _lib.P],
})


def available() -> bool:
    return torch.cuda.is_available()


def sample(logits: torch.Tensor, temperature: float, top_p: Optional[float], top_k: Optional[int], seed: int, step: int,
           want_logprob: bool = False, out_tokens: Optional[torch.Tensor] = None,
           out_logprobs: Optional[torch.Tensor] = None, step_tensor: Optional[torch.Tensor] = None,
           softcap: float = 0.0, forbidden: Optional[torch.Tensor] = None):
    """logits fp32 [B, V] on CUDA -> (tokens int64 [B], logprobs fp32 [B] | None).

    `softcap` > 0 applies cap * tanh(z / cap) and `forbidden` (int32 ids on the device) removes tokens from the
    distribution inside the kernel; both rewrite `logits` in place."""
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    B, V = logits.shape
    tok = out_tokens if out_tokens is not None else torch.empty(B, dtype=torch.int64, device=logits.device)
    lp = out_logprobs if out_logprobs is not None else (
        torch.empty(B, dtype=torch.float32, device=logits.device) if want_logprob else None)
    if (softcap and softcap > 0) or forbidden is not None:
        if forbidden is not None:
            assert forbidden.is_cuda and forbidden.dtype == torch.int32 and forbidden.is_contiguous()
        rc = _lib.cuda().tb_sample_ex(logits.data_ptr(), logits.stride(0), B, V, float(temperature or 0.0), int(top_k or 0),
                                      float(top_p if top_p is not None else 1.0), int(seed) & 0xFFFFFFFFFFFFFFFF, int(step),
                                      _lib.ptr(step_tensor), tok.data_ptr(), _lib.ptr(lp), float(softcap or 0.0),
                                      _lib.ptr(forbidden), 0 if forbidden is None else forbidden.numel(), _lib.stream_ptr())
        _lib.check(rc, "tb_sample_ex")
        K._count()
        return tok, lp
    rc = _lib.cuda().tb_sample(logits.data_ptr(), logits.stride(0), B, V, float(temperature or 0.0), int(top_k or 0),
                               float(top_p if top_p is not None else 1.0), int(seed) & 0xFFFFFFFFFFFFFFFF, int(step),
                               _lib.ptr(step_tensor), tok.data_ptr(), _lib.ptr(lp), _lib.stream_ptr())
    _lib.check(rc, "tb_sample")
    K._count()
    return tok, lp
