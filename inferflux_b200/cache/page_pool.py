"""A pool of equally sized pages with a free list.

The reference keeps its page bookkeeping on the host only
(runtime/kv_cache/paged_kv_cache.cpp:39-66 allocation, :90-112 reference
counts) while its kernels read a dense per-sequence buffer
(runtime/backends/cuda/native/kv_cache_gpu.cu:32-38).  Here the pool's page
numbers are the ones the kernels index through block tables.  Pages are not
cleared when they are given back: a request only ever reads positions it has
written, so stale contents are never visible.
"""
from __future__ import annotations

from typing import Iterable, List


class OutOfPages(RuntimeError):
    """Raised when a pool cannot hand out the pages asked for; nothing is
    taken in that case."""

    def __init__(self, wanted: int, free: int, group: int = 0):
        super().__init__(f"cache group {group}: {wanted} page(s) wanted, {free} free")
        self.wanted, self.free, self.group = wanted, free, group


class PagePool:
    def __init__(self, num_pages: int, group: int = 0):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self.group = group
        # last freed = first reused, so reuse shows up early
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages
        self.allocations = 0
        self.reuses = 0
        self._ever_used = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(n, len(self._free), self.group)
        out = []
        for _ in range(n):
            p = self._free.pop()
            assert not self._held[p], f"page {p} handed out twice"
            self._held[p] = True
            if self._ever_used[p]:
                self.reuses += 1
            self._ever_used[p] = True
            out.append(p)
        self.allocations += n
        return out

    def free(self, pages: Iterable[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not of this pool")
            if not self._held[p]:
                raise ValueError(f"page {p} freed twice (or never handed out)")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """No page lost, none both free and held, none twice in the free list."""
        assert len(set(self._free)) == len(self._free), "a page is twice in the free list"
        for p in self._free:
            assert not self._held[p], f"page {p} is free and held"
        assert sum(self._held) + len(self._free) == self.num_pages, "a page was lost"
