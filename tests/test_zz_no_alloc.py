"""The allocation-free attention-backward entry point, called through its exported C symbol.

Some users of the CUDA library cannot allocate device memory when they call it (a stream capture in
progress, a device-memory pool owned by someone else, a C host without torch). For them
`tb_attn_bwd_noalloc` keeps its scratch inside the library. This test drives that symbol directly with
ctypes -- no Python wrapper in between -- and compares it with the regular entry point, twice in a row
because the built-in scratch is shared between calls and keeps old contents. A plain PyTorch fp32 attention
is the second reference, so that the two entry points cannot be wrong together. "Allocates nothing" is checked
on the driver's own count of free device memory (`cudaMemGetInfo`), which also sees a raw `cudaMalloc` that
torch's allocator statistics would miss.

The file name sorts last on purpose: a run that stops at the first failure has then already executed
every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from tunix_b200 import _build
    lib = ctypes.CDLL(str(_build.build_cuda()))
    fn = lib.tb_attn_bwd_noalloc
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp] * 9 + [i] * 6 + [f, f, i, i, vp, vp]
    fn.restype = i
    lib.tb_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()


def _case(seed, B, T, N, KH, H):
    torch.manual_seed(seed)
    q = torch.randn(B, T, N, H, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, T, KH, H, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, T, KH, H, device="cuda", dtype=torch.bfloat16)
    do = torch.randn(B, T, N, H, device="cuda", dtype=torch.bfloat16)
    return q, k, v, do


def test_noalloc_attention_backward_matches_regular_entry_point_twice():
    from tunix_b200 import _lib
    from tunix_b200.ops import kernels as K
    from tunix_b200.ops import reference as R
    lib, fn = _symbol()
    first = True
    status = _lib.status_buffer()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second must not see leftovers of the first
    for seed, shape in ((0, (2, 256, 4, 2, 128)), (1, (1, 320, 2, 1, 64))):
        B, T, N, KH, H = shape
        q, k, v, do = _case(seed, *shape)
        scale = 1.0 / math.sqrt(H)
        o, lse = K.attn_fwd(q, k, v, scale=scale, causal=True)
        dq_ref, dk_ref, dv_ref = K.attn_bwd(do, q, k, v, o, lse, scale=scale, causal=True)
        # the same gradients from PyTorch autograd in fp32
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        of = R.attention_ref(qf, kf, vf, scale=scale, causal=True)
        of.backward(do.float())
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if first:
            # the first call on a device looks the scratch addresses up; do it before measuring
            rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                    dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, T, T, N, KH, H, scale, 0.0, 1, 0,
                    status.data_ptr(), stream)
            assert rc == 0, lib.tb_noalloc_last_error()
            first = False
            dq.zero_(), dk.zero_(), dv.zero_()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, T, T, N, KH, H, scale, 0.0, 1, 0,
                status.data_ptr(), stream)
        assert rc == 0, lib.tb_noalloc_last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_allocated() == before
        assert free_after >= free_before, (free_before, free_after)     # nothing was taken from the device
        _lib.raise_if_kernel_error()
        for got, same_math, fp32 in ((dq, dq_ref, qf.grad), (dk, dk_ref, kf.grad), (dv, dv_ref, vf.grad)):
            assert _rel(got, same_math) < 3e-2
            assert _rel(got, fp32) < 3e-2
            # element-wise as well: a few wrong elements cannot hide in a norm
            assert torch.allclose(got.float(), fp32, atol=0.06 * fp32.abs().max().item(), rtol=0.05)


def test_noalloc_rejects_oversized_problem():
    lib, fn = _symbol()
    # 8 * 4096 * 32 * 128 elements is far beyond the 4 Mi-element scratch: refused before any launch
    rc = fn(0, 0, 0, 0, 0, 0, 0, 0, 0, 8, 4096, 4096, 32, 8, 128, 0.1, 0.0, 1, 0, 0, 0)
    assert rc == -11
    assert b"too large" in lib.tb_noalloc_last_error()
