"""Host-side page management of a paged KV cache with prefix caching
(tunix/experimental/generate/single_type_kv_cache_manager.py:42-395, tiered_page_pool.py:39-534).

`PagePool` is a free list over page indices with double-free checks. `KVCacheManager` (one per attention type:
global, or sliding with `window_size`) maps `request_id -> [Page | None]`:

  * only FULL pages are hashed; the hash of page i chains the hash of page i-1 with the page's token ids, so a
    hit on page i implies the whole prefix matches;
  * on a hit the request re-points to the cached page (ref count + 1) and returns its own page to the pool;
  * released pages that were hashed stay resident, unreferenced, in LRU order and are evicted only when the
    pool runs dry; pages that were never hashed are freed at once;
  * sliding-window managers release pages that lie wholly below `num_completed_tokens - window`;
  * the longest cached prefix is the leading run of hits (global) or, for a sliding window, the right-most
    position where every page of the window hits (earlier pages are then `None`).

The device side (page writes, paged attention) lives in `csrc/decode.cu`; the page table this manager maintains
is what `generate/engine.py` uploads."""
from __future__ import annotations

import collections
import dataclasses
import hashlib
from typing import Optional, Sequence


class PagePoolError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = collections.deque(range(num_pages))
        self._in_use: set = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int = 1) -> list:
        if n > len(self._free):
            raise PagePoolError(f"asked for {n} pages, {len(self._free)} free")
        out = [self._free.popleft() for _ in range(n)]
        self._in_use.update(out)
        return out

    def free(self, page_ids: Sequence[int]) -> None:
        for p in page_ids:
            if p not in self._in_use:
                raise PagePoolError(f"page {p} is not in use (double free?)")
        for p in page_ids:
            self._in_use.discard(p)
            self._free.append(p)


@dataclasses.dataclass
class Page:
    page_id: int
    ref_count: int = 1
    prefix_hash: Optional[bytes] = None
    is_freed: bool = False


def _chain_hash(prev: Optional[bytes], token_ids: Sequence[int]) -> bytes:
    h = hashlib.blake2b(digest_size=16)
    h.update(prev or b"\x00" * 16)
    h.update(b"".join(int(t).to_bytes(4, "little", signed=True) for t in token_ids))
    return h.digest()


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


class KVCacheManager:
    def __init__(self, pool: PagePool, page_size: int, window_size: Optional[int] = None, enable_prefix_caching: bool = True):
        self.pool, self.page_size, self.window_size = pool, page_size, window_size
        self.enable_prefix_caching = enable_prefix_caching
        self._req: dict = {}                                   # request id -> [Page | None]
        self._by_hash: dict = {}                               # prefix hash -> Page
        self._lru: "collections.OrderedDict[int, Page]" = collections.OrderedDict()   # unreferenced cached pages

    @property
    def pages_in_window(self) -> Optional[int]:
        return None if self.window_size is None else cdiv(self.window_size - 1, self.page_size) + 1

    # ------------------------------------------------------------------ pool with eviction
    def _allocate(self, n: int) -> list:
        while self.pool.num_free < n and self._lru:
            _, victim = self._lru.popitem(last=False)          # least recently released first
            self._by_hash.pop(victim.prefix_hash, None)
            victim.is_freed = True
            self.pool.free([victim.page_id])
        return [Page(p) for p in self.pool.allocate(n)]

    def _unref(self, page: Page) -> None:
        page.ref_count -= 1
        if page.ref_count > 0:
            return
        if page.prefix_hash is not None and self._by_hash.get(page.prefix_hash) is page:
            self._lru[page.page_id] = page                      # stays cached until the pool needs it
        else:
            page.is_freed = True
            self.pool.free([page.page_id])

    def _ref(self, page: Page) -> None:
        if page.ref_count == 0:
            self._lru.pop(page.page_id, None)
        page.ref_count += 1

    # ----------------------------------------------------------------------------- requests
    def find_longest_cache_hit(self, token_ids: Sequence[int]) -> list:
        """Pages (or None) covering the longest cached prefix of `token_ids`; whole pages only."""
        if not self.enable_prefix_caching:
            return []
        hits, prev = [], None
        for i in range(len(token_ids) // self.page_size):
            prev = _chain_hash(prev, token_ids[i * self.page_size:(i + 1) * self.page_size])
            hits.append(self._by_hash.get(prev))
        if self.window_size is None:
            n = 0
            while n < len(hits) and hits[n] is not None:
                n += 1
            return hits[:n]
        w = self.pages_in_window
        for end in range(len(hits), 0, -1):                     # right-most fully hit window
            lo = max(0, end - w)
            if all(h is not None for h in hits[lo:end]):
                return [None] * lo + hits[lo:end]
        return []

    def allocate_for_request(self, request_id: str, token_ids: Sequence[int], num_new_tokens: int = 0) -> tuple:
        """Gives the request pages for len(token_ids) + num_new_tokens tokens. Returns (pages, cached tokens)."""
        if request_id in self._req:
            raise KeyError(f"request {request_id} already has pages")
        cached = self.find_longest_cache_hit(token_ids)
        for p in cached:
            if p is not None:
                self._ref(p)
        need = cdiv(len(token_ids) + num_new_tokens, self.page_size) - len(cached)
        try:
            fresh = self._allocate(max(need, 0))
        except PagePoolError:
            for p in cached:
                if p is not None:
                    self._unref(p)
            raise
        self._req[request_id] = list(cached) + fresh
        return self._req[request_id], len(cached) * self.page_size

    def append_pages(self, request_id: str, total_tokens: int) -> list:
        pages = self._req[request_id]
        need = cdiv(total_tokens, self.page_size) - len(pages)
        if need > 0:
            pages += self._allocate(need)
        return pages

    def cache_full_pages(self, request_id: str, token_ids: Sequence[int], num_completed_tokens: int) -> None:
        """Hash every page that is now full. A page whose hash is already cached is swapped for the cached one."""
        if not self.enable_prefix_caching:
            return
        pages = self._req[request_id]
        prev = None
        for i in range(min(num_completed_tokens, len(token_ids)) // self.page_size):
            prev = _chain_hash(prev, token_ids[i * self.page_size:(i + 1) * self.page_size])
            page = pages[i]
            if page is None or page.prefix_hash is not None:
                continue
            other = self._by_hash.get(prev)
            if other is not None and other is not page:
                self._ref(other)
                pages[i] = other
                page.is_freed = True
                self.pool.free([page.page_id])
            else:
                page.prefix_hash = prev
                self._by_hash[prev] = page

    def release_out_of_window(self, request_id: str, num_completed_tokens: int) -> int:
        if self.window_size is None:
            return 0
        pages = self._req[request_id]
        last_dead = (num_completed_tokens - self.window_size) // self.page_size      # pages [0, last_dead) are dead
        n = 0
        for i in range(max(0, min(last_dead, len(pages)))):
            if pages[i] is not None:
                self._unref(pages[i])
                pages[i] = None
                n += 1
        return n

    def free_request(self, request_id: str) -> None:
        for p in reversed(self._req.pop(request_id)):           # tail pages first: the LRU keeps prefixes longest
            if p is not None:
                self._unref(p)

    def page_table(self, request_id: str, pad_to: int, fill: int = -1) -> list:
        ids = [fill if p is None else p.page_id for p in self._req[request_id]]
        return ids + [fill] * (pad_to - len(ids))
