"""A pool of cache pages: a FIFO ring of free pages and a reference count per page.

Free pages form a FIFO ring that starts as ``0 .. N-1``; pages given back are
queued in the order they are released, so the order in which pages are used again
is a pure function of the request trace (the reference's rule,
src/kv_cache/paged.cpp:139-188).  A page may be held by several requests once a
prefix is shared (src/kv_cache/paged.cpp:535-620); it returns to the ring when its
last holder lets go.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Iterable, List


class OutOfPages(RuntimeError):
    """The pool cannot serve the pages asked for; nothing was taken."""


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: Deque[int] = deque(range(self.num_pages))
        self._refs: List[int] = [0] * self.num_pages
        self.allocation_count = 0
        self.release_count = 0
        self.reuse_count = 0          # allocations of a page that was used before
        self._ever_used = [False] * self.num_pages
        self.peak_in_use = 0

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def pages_in_use(self) -> int:
        return self.num_pages - len(self._free)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def allocate(self, count: int) -> List[int]:
        """Take ``count`` pages from the head of the ring, or raise and take none."""
        if count < 0:
            raise ValueError("page count must not be negative")
        if count > len(self._free):
            raise OutOfPages(f"{count} pages asked for, {len(self._free)} free")
        pages = [self._free.popleft() for _ in range(count)]
        for page in pages:
            assert self._refs[page] == 0, f"free page {page} has holders"
            self._refs[page] = 1
            if self._ever_used[page]:
                self.reuse_count += 1
            self._ever_used[page] = True
        self.allocation_count += count
        self.peak_in_use = max(self.peak_in_use, self.pages_in_use)
        return pages

    def share(self, pages: Iterable[int]) -> None:
        """One more holder for each page (prefix sharing)."""
        pages = list(pages)
        for page in pages:
            if self._refs[page] <= 0:
                raise RuntimeError(f"page {page} is free and cannot be shared")
        for page in pages:
            self._refs[page] += 1

    def release(self, pages: Iterable[int]) -> int:
        """Drop one holder per page, in order; return how many pages became free."""
        freed = 0
        for page in pages:
            if self._refs[page] <= 0:
                raise RuntimeError(f"page {page} released more often than it was taken")
            self._refs[page] -= 1
            if self._refs[page] == 0:
                self._free.append(page)
                freed += 1
        self.release_count += freed
        return freed

    def last_freed(self, count: int) -> List[int]:
        """The ``count`` pages that became free most recently (the tail of the ring)."""
        if count <= 0:
            return []
        return list(self._free)[-count:]

    def check(self) -> None:
        """Every page is either free exactly once or held; raises AssertionError otherwise."""
        free = list(self._free)
        assert len(free) == len(set(free)), "a page is in the free ring twice"
        for page in range(self.num_pages):
            in_ring = page in set(free)
            assert in_ring == (self._refs[page] == 0), f"page {page}: ring/refcount disagree"
            assert self._refs[page] >= 0
