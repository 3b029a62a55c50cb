"""Host model of the device-side flag protocols, with threads standing in for ranks.

The flag barrier of `csrc/comm.cu` (`symm_barrier_kernel`) is restated here word for word on a shared integer array,
so that its logic (who writes which word, the wrap-safe epoch comparison, what a rank that never arrives does to
the others) is exercised on the CPU, where thread schedules can be made adversarial and a wait that runs out costs
nothing. Kernels that wait on one another must not be run as separate launches on one GPU, so this model is also the
only place where more ranks than GPUs can be tried.

Layout, as on the device: rank r owns `world * slots` 32-bit words; slot s uses words `[s * world, (s + 1) * world)`;
word `s * world + p` of rank r is written ONLY by rank p. A rank entering barrier (slot, epoch) stores `epoch` into
its word at every peer (release), then spins on its own words until each holds a value not older than `epoch`
(`(int32)(word - epoch) >= 0`, which survives the 32-bit wrap), or until the time limit, after which it records
status 4, the peer it was waiting for and the epoch, and returns."""
from __future__ import annotations

import threading
import time

import numpy as np

ST_TIMEOUT_FLAG = 4


def _not_older(word: int, epoch: int) -> bool:
    d = (int(word) - int(epoch)) & 0xFFFFFFFF
    return d < 0x80000000                                   # (int32)(word - epoch) >= 0


class FlagBarrierModel:
    def __init__(self, world: int, slots: int = 8):
        self.world, self.slots = world, slots
        self.flags = np.zeros((world, slots * world), np.uint32)      # flags[r] is rank r's symmetric buffer
        self.status = np.zeros((world, 3), np.int64)                   # per rank: code, peer, epoch
        self._epochs = [[0] * slots for _ in range(world)]

    def set_epoch(self, value: int) -> None:
        """Start every rank's epoch counters (and the flag words) at `value`, e.g. just below the 32-bit wrap."""
        self.flags[:] = np.uint32(value & 0xFFFFFFFF)
        self._epochs = [[value] * self.slots for _ in range(self.world)]

    def wait(self, rank: int, slot: int = 0, timeout_s: float = 5.0, yield_fn=None) -> bool:
        """One barrier call of `rank`; True when every peer arrived, False after the time limit (status recorded)."""
        self._epochs[rank][slot] += 1
        epoch = self._epochs[rank][slot] & 0xFFFFFFFF
        w = self.world
        for p in range(w):                                  # thread p of the kernel publishes to peer p ...
            if yield_fn is not None:
                yield_fn()
            self.flags[p, slot * w + rank] = epoch
        t0 = time.monotonic()
        for p in range(w):                                  # ... and waits for peer p's word in its own buffer
            while not _not_older(self.flags[rank, slot * w + p], epoch):
                if time.monotonic() - t0 > timeout_s:
                    if self.status[rank, 0] == 0:
                        self.status[rank] = (ST_TIMEOUT_FLAG, p, epoch)
                    return False
                if yield_fn is not None:
                    yield_fn()
                else:
                    time.sleep(0)
        return True


def run_ranks(world: int, body, timeout_s: float = 60.0) -> list:
    """Run `body(rank)` on one thread per rank; returns the results in rank order, re-raising the first failure."""
    out: list = [None] * world
    errs: list = []

    def run(r):
        try:
            out[r] = body(r)
        except BaseException as e:
            errs.append(e)
    ts = [threading.Thread(target=run, args=(r,), daemon=True) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout_s)
    if any(t.is_alive() for t in ts):
        raise TimeoutError("a rank thread is still running")
    if errs:
        raise errs[0]
    return out
