"""KV pages on two tiers: device memory and pinned host memory
(tunix/experimental/generate/tiered_page_pool.py:32-534).

Callers hold stable LOGICAL page ids; the pool tracks where each page lives (tier and physical index) and moves
pages between the tiers in batches. One pool serves several caches of the same geometry (for instance the K and V
pools of every layer): each is a named partition, and a logical page owns the same physical index in all of them, so
one `offload` moves the page's slice of every partition.

A move gathers (offload) or scatters (load) on the DEVICE through one contiguous block per partition and crosses
the link with one copy per run of neighbouring host slots, straight out of / into the pinned host pool: no staging
on the host, no CPU scatter, and, because the free lists hand out the lowest indices first, usually a single large
copy per partition instead of a copy per page, which is what a PCIe / NVLink-C2C link wants. Measured on one B200
(`python -m tunix_b200.experimental.generate.tiered_page_pool`, 1024 pages of 256 KiB over two partitions, CUDA
events): offload 51 GB/s, load 48 GB/s, whether the device pages are neighbours or not. On a CUDA device the copies run on the pool's own stream from / to pinned host
memory and the caller's stream waits on an event, so that decode steps which do not touch the moved pages overlap
with the transfer.

The host-side page tables (`kv_cache_manager.KVCacheManager`) decide WHICH pages to evict; this class only moves
them and keeps the books."""
from __future__ import annotations

import enum
from typing import Mapping, Optional, Sequence

import torch


class PageLocation(enum.Enum):
    DEVICE = "device"
    HOST = "host"


class TieredPoolError(RuntimeError):
    pass


class _Tier:
    """Free list over the physical indices of one tier, with double-free checks."""

    def __init__(self, n: int):
        self.n = n
        self._free = list(range(n - 1, -1, -1))
        self._used: set = set()

    def num_free(self) -> int:
        return len(self._free)

    def take(self, k: int) -> list:
        if k > len(self._free):
            raise TieredPoolError(f"asked for {k} pages, {len(self._free)} free")
        if k > 1:
            self._free.sort(reverse=True)                   # lowest indices first: neighbours, so copies coalesce into runs
        out = [self._free.pop() for _ in range(k)]
        self._used.update(out)
        return out

    def give(self, idx: Sequence[int]) -> None:
        for i in idx:
            if i not in self._used:
                raise TieredPoolError(f"physical page {i} is not in use")
            self._used.discard(i)
            self._free.append(i)


class TieredPagePool:
    def __init__(self, partitions: Sequence[str], page_shape: Sequence[int], dtype: torch.dtype, num_device_pages: int,
                 num_host_pages: int, device: Optional[torch.device] = None,
                 device_pages: Optional[Mapping[str, torch.Tensor]] = None):
        """`device_pages` adopts existing pools (e.g. the engine's K / V page pools) instead of allocating new ones;
        each must be `[num_device_pages, *page_shape]`."""
        if not partitions:
            raise ValueError("at least one partition")
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.page_shape, self.dtype = tuple(page_shape), dtype
        self._cuda = self.device.type == "cuda"
        if device_pages is not None:
            for name in partitions:
                t = device_pages[name]
                if tuple(t.shape) != (num_device_pages, *self.page_shape) or t.dtype != dtype:
                    raise ValueError(f"partition {name!r}: expected {(num_device_pages, *self.page_shape)} {dtype}, "
                                     f"got {tuple(t.shape)} {t.dtype}")
            self.dev = {n: device_pages[n] for n in partitions}
        else:
            self.dev = {n: torch.zeros((num_device_pages, *self.page_shape), dtype=dtype, device=self.device) for n in partitions}
        self.host = {n: torch.zeros((num_host_pages, *self.page_shape), dtype=dtype, pin_memory=self._cuda) for n in partitions}
        self._dev_tier, self._host_tier = _Tier(num_device_pages), _Tier(num_host_pages)
        self._where: dict = {}                              # logical id -> (PageLocation, physical index)
        self._next_id = 0
        self._stream = torch.cuda.Stream(self.device) if self._cuda else None
        self.bytes_offloaded = self.bytes_loaded = 0

    # ------------------------------------------------------------------ books
    @property
    def num_free_device_pages(self) -> int:
        return self._dev_tier.num_free()

    @property
    def num_free_host_pages(self) -> int:
        return self._host_tier.num_free()

    def page_location(self, page_id: int) -> Optional[PageLocation]:
        e = self._where.get(page_id)
        return e[0] if e else None

    def page_idx(self, page_id: int) -> Optional[int]:
        e = self._where.get(page_id)
        return e[1] if e else None

    def device_indices(self, page_ids: Sequence[int]) -> list:
        """Physical device indices for a page table; raises if a page is not resident."""
        out = []
        for p in page_ids:
            loc, idx = self._entry(p)
            if loc is not PageLocation.DEVICE:
                raise TieredPoolError(f"page {p} is on the host; load it first")
            out.append(idx)
        return out

    def _entry(self, page_id: int):
        e = self._where.get(page_id)
        if e is None:
            raise TieredPoolError(f"unknown page {page_id}")
        return e

    def allocate_device_pages(self, n: int) -> list:
        phys = self._dev_tier.take(n)
        ids = list(range(self._next_id, self._next_id + n))
        self._next_id += n
        for i, p in zip(ids, phys):
            self._where[i] = (PageLocation.DEVICE, p)
        return ids

    def free(self, page_ids: Sequence[int]) -> None:
        ids = list(page_ids)
        if len(set(ids)) != len(ids):
            raise TieredPoolError("duplicate page ids in free()")
        entries = [self._entry(p) for p in ids]            # validate everything before changing anything
        for p, (loc, idx) in zip(ids, entries):
            (self._dev_tier if loc is PageLocation.DEVICE else self._host_tier).give([idx])
            del self._where[p]

    # ------------------------------------------------------------------ moves
    def _move(self, ids: Sequence[int], src_loc: PageLocation) -> int:
        ids = list(ids)
        if len(set(ids)) != len(ids):
            raise TieredPoolError("duplicate page ids in a move")
        src_idx = []
        for p in ids:
            loc, idx = self._entry(p)
            if loc is not src_loc:
                raise TieredPoolError(f"page {p} is already on the {('host', 'device')[src_loc is PageLocation.HOST]}")
            src_idx.append(idx)
        if not ids:
            return 0
        to_host = src_loc is PageLocation.DEVICE
        dst_tier, src_tier = (self._host_tier, self._dev_tier) if to_host else (self._dev_tier, self._host_tier)
        dst_idx = dst_tier.take(len(ids))                   # raises before anything moved when the target tier is full
        src_pool, dst_pool = (self.dev, self.host) if to_host else (self.host, self.dev)
        moved = 0
        if self._cuda:
            cur = torch.cuda.current_stream(self.device)
            self._stream.wait_stream(cur)                   # the pages' last writers have been enqueued on `cur`
        ctx = torch.cuda.stream(self._stream) if self._cuda else _null()
        nb = self._cuda
        with ctx:
            if to_host:
                si_d = torch.as_tensor(src_idx, dtype=torch.long, device=self.device)
                for name in src_pool:
                    block = src_pool[name].index_select(0, si_d)                     # gather on the device: one contiguous block
                    for pos, a, n in _runs(dst_idx):                                 # one device -> host copy per run of host slots,
                        dst_pool[name][a:a + n].copy_(block[pos:pos + n], non_blocking=nb)   # straight into the pinned pool
                    if nb:
                        block.record_stream(self._stream)
                    moved += block.numel() * block.element_size()
            else:
                di_d = torch.as_tensor(dst_idx, dtype=torch.long, device=self.device)
                for name in src_pool:
                    block = torch.empty((len(ids), *self.page_shape), dtype=self.dtype, device=self.device)
                    for pos, a, n in _runs(src_idx):                                 # one host -> device copy per run, from the pinned pool
                        block[pos:pos + n].copy_(src_pool[name][a:a + n], non_blocking=nb)
                    dst_pool[name].index_copy_(0, di_d, block)                       # scatter on the device
                    if nb:
                        block.record_stream(self._stream)
                    moved += block.numel() * block.element_size()
            if nb and to_host:
                self._stream.synchronize()                  # the host pool is read by whoever loads next, possibly on the CPU
        if self._cuda:
            torch.cuda.current_stream(self.device).wait_stream(self._stream)
        src_tier.give(src_idx)
        dst_loc = PageLocation.HOST if to_host else PageLocation.DEVICE
        for p, i in zip(ids, dst_idx):
            self._where[p] = (dst_loc, i)
        return moved

    def offload(self, page_ids: Sequence[int]) -> None:
        """Move resident pages to the host tier; their device slots become free."""
        self.bytes_offloaded += self._move(page_ids, PageLocation.DEVICE)

    def load(self, page_ids: Sequence[int]) -> None:
        """Bring host pages back; they may land on different physical device indices than before."""
        self.bytes_loaded += self._move(page_ids, PageLocation.HOST)


def _runs(idx: Sequence[int]):
    """(position in the list, first index, length) for every run of consecutive indices."""
    out, start = [], 0
    for i in range(1, len(idx) + 1):
        if i == len(idx) or idx[i] != idx[i - 1] + 1:
            out.append((start, idx[start], i - start))
            start = i
    return out


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def _bench(pages: int = 2048, move: int = 1024, iters: int = 5) -> None:
    """python -m tunix_b200.experimental.generate.tiered_page_pool : offload / load bandwidth on cuda:0."""
    dev = torch.device("cuda")
    pool = TieredPagePool(["k", "v"], (64, 8, 128), torch.bfloat16, pages, move, device=dev)
    ids = pool.allocate_device_pages(pages)
    for contiguous in (True, False):
        pick = ids[:move] if contiguous else ids[::2][:move]
        for _ in range(2):
            pool.offload(pick), pool.load(pick)
        t_off = t_on = 0.0
        for _ in range(iters):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            torch.cuda.synchronize()
            e[0].record(); pool.offload(pick); e[1].record(); pool.load(pick); e[2].record()
            torch.cuda.synchronize()
            t_off += e[0].elapsed_time(e[1]); t_on += e[1].elapsed_time(e[2])
        nbytes = move * 2 * 64 * 8 * 128 * 2
        print(f"{'neighbouring' if contiguous else 'every other'} device pages, {move} x {nbytes // move // 1024} KiB: "
              f"offload {nbytes * iters / t_off / 1e6:.1f} GB/s, load {nbytes * iters / t_on / 1e6:.1f} GB/s")


if __name__ == "__main__":
    _bench()
