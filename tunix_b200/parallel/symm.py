"""Symmetric device memory: buffers of identical size on every rank, each mapped into every peer.

Allocation and handle exchange use `torch.distributed._symmetric_memory` (CUDA VMM allocations whose
handles travel over the process group's store); what comes back is, per buffer, the list of device
pointers under which THIS rank can address EVERY rank's copy. Our own kernels (csrc/comm.cu) take that
pointer table and move data with peer loads over NVLink. NVLS multicast is deliberately not used by any
kernel of this package: a rank that dies while bound to a multicast object can fault its peers.

On CPU (gloo) or a single rank the "symmetric" buffer is an ordinary tensor and the pointer table has
one entry, so the same call sites work everywhere.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib

_lib.register_cuda_sigs({
    "tb_symm_barrier": [_lib.P, _lib.I, _lib.I, _lib.I, ctypes.c_uint, _lib.LL, _lib.P, _lib.P],
})


class SymmBuffer:
    def __init__(self, tensor: torch.Tensor, ptrs: list[int], rank: int, world: int, handle=None):
        self.tensor, self.ptrs, self.rank, self.world, self.handle = tensor, ptrs, rank, world, handle
        arr = (ctypes.c_void_p * 8)(*([p for p in ptrs] + [None] * (8 - len(ptrs))))
        self._c_array = arr  # keep alive; passed as `const void* const*`

    @property
    def c_ptrs(self):
        return ctypes.cast(self._c_array, ctypes.c_void_p)

    def peer_tensor(self, peer: int) -> torch.Tensor:
        """A tensor view of a peer's copy (only through torch symmetric memory)."""
        if self.handle is None or peer == self.rank:
            return self.tensor
        return self.handle.get_buffer(peer, tuple(self.tensor.shape), self.tensor.dtype)


def symm_available(group=None) -> bool:
    if not (dist.is_initialized() and torch.cuda.is_available()):
        return False
    if dist.get_world_size(group) <= 1:
        return False
    try:
        import importlib
        importlib.import_module("torch.distributed._symmetric_memory")
        return "nccl" in str(dist.get_backend(group))
    except Exception:
        return False


def symm_empty(numel: int, dtype: torch.dtype, device, group=None, zero: bool = True) -> SymmBuffer:
    """Collective: every rank of `group` must call with the same size."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if world > 1 and torch.device(device).type == "cuda":
        import torch.distributed._symmetric_memory as sm
        t = sm.empty(numel, dtype=dtype, device=device)
        if zero:
            t.zero_()
        pg = group if group is not None else dist.group.WORLD
        h = sm.rendezvous(t, pg)
        ptrs = [int(p) for p in h.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier(group)
        return SymmBuffer(t, ptrs, rank, world, h)
    t = torch.zeros(numel, dtype=dtype, device=device) if zero else torch.empty(numel, dtype=dtype, device=device)
    return SymmBuffer(t, [t.data_ptr()], 0, 1, None)


class SymmBarrier:
    """Device-side flag barrier over symmetric memory with a bounded wait.

    `wait(stream)` enqueues one tiny kernel: it publishes this rank's epoch to every peer, then spins
    (at most `timeout_ms`) until every peer's epoch arrived. On expiry the kernel writes code 4 to the
    status word and returns; `_lib.raise_if_kernel_error()` turns that into a Python exception.
    """

    SLOTS = 8

    def __init__(self, device, group=None, timeout_ms: int = 20000):
        self.buf = symm_empty(self.SLOTS * 8, torch.int32, device, group, zero=True)
        self.epochs = [0] * self.SLOTS
        self.timeout_ms = timeout_ms

    def wait(self, slot: int = 0, timeout_ms: Optional[int] = None) -> None:
        b = self.buf
        if b.world == 1:
            return
        self.epochs[slot] += 1
        status = _lib.status_buffer(b.tensor.device)
        rc = _lib.cuda().tb_symm_barrier(b.c_ptrs, b.rank, b.world, slot, self.epochs[slot],
                                         int(timeout_ms or self.timeout_ms), status.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "tb_symm_barrier")
