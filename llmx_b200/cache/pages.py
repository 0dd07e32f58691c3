"""Page bookkeeping: a pool of page ids and one request's block table over it.

The protocol is the reference's (src/model/kv_cache.hpp:14-67 for the pool,
:71-179 for a sequence): pages for a step are *prepared* before the step
writes, *committed* after the whole step has been enqueued, and *aborted* when
it fails, which returns exactly the pages the failed step took.  What differs:
a block table here may belong to a group of layers that keeps only a window of
keys, and then gives back the pages the window has passed at every commit.
"""
from __future__ import annotations

from typing import List, Optional


class CacheExhausted(RuntimeError):
    """The page pool cannot cover the tokens asked for."""


class PagePool:
    """Page ids 0..num_pages-1 with reference counts and a LIFO free list."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("a pool cannot have a negative number of pages")
        self.num_pages = int(num_pages)
        self._refs: List[int] = [0] * self.num_pages
        # Lowest ids are handed out first from a fresh pool.
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def refs(self, page: int) -> int:
        return self._refs[page]

    def alloc(self) -> int:
        if not self._free:
            raise CacheExhausted(
                f"KV cache: all {self.num_pages} pages are in use; the run needs more tokens than the cache was made for")
        page = self._free.pop()
        assert self._refs[page] == 0
        self._refs[page] = 1
        return page

    def retain(self, page: int) -> None:
        if self._refs[page] == 0:
            raise RuntimeError(f"KV cache: retain of free page {page}")
        self._refs[page] += 1

    def release(self, page: int) -> None:
        if not 0 <= page < self.num_pages or self._refs[page] == 0:
            raise RuntimeError(f"KV cache: page {page} released twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def check(self) -> None:
        """Every page is either free exactly once or referenced; none is lost."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (self._refs[p] == 0) != (p in seen):
                raise AssertionError(f"page {p}: refs {self._refs[p]} but free={p in seen}")


RELEASED = -1


class BlockTable:
    """One request's pages in one group: logical page number -> page id.

    `window`: None keeps every key; W keeps, for a query at position p, the
    keys p-W+1..p, so once `length` tokens are committed no later query needs a
    key below length-W+1 and the pages wholly below that are given back (their
    entries become RELEASED and are never read again).
    """

    def __init__(self, pool: PagePool, page_size: int, window: Optional[int] = None):
        if page_size <= 0:
            raise ValueError("a page holds at least one token")
        if window is not None and window <= 0:
            raise ValueError("a window holds at least one key")
        self.pool = pool
        self.page_size = int(page_size)
        self.window = window
        self.pages: List[int] = []
        self.length = 0          # committed tokens
        self.pending = 0         # prepared, not yet committed
        self._first_live = 0     # logical pages below this were given back
        self._taken_by_prepare = 0

    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    @property
    def held_pages(self) -> int:
        return len(self.pages) - self._first_live

    def prepare(self, n: int) -> None:
        """Make positions [length, length+n) addressable; on exhaustion give back what this call took."""
        if self.pending:
            raise RuntimeError("KV cache: a step is already in progress for this request")
        if n < 0:
            raise ValueError("cannot prepare a negative number of tokens")
        need = self.pages_for(self.length + n)
        taken = 0
        try:
            while len(self.pages) < need:
                self.pages.append(self.pool.alloc())
                taken += 1
        except CacheExhausted:
            for _ in range(taken):
                self.pool.release(self.pages.pop())
            raise
        self._taken_by_prepare = taken
        self.pending = n

    def commit(self) -> None:
        self.length += self.pending
        self.pending = 0
        self._taken_by_prepare = 0
        self._release_passed()

    def abort(self) -> None:
        """Undo a prepare: the committed history stays, the pages taken for the step go back."""
        keep = max(self.pages_for(self.length), self._first_live)
        while len(self.pages) > keep:
            self.pool.release(self.pages.pop())
        self.pending = 0
        self._taken_by_prepare = 0

    def _release_passed(self) -> None:
        if self.window is None:
            return
        lowest_needed = self.length - self.window + 1
        if lowest_needed <= 0:
            return
        upto = min(lowest_needed // self.page_size, len(self.pages))
        for i in range(self._first_live, upto):
            self.pool.release(self.pages[i])
            self.pages[i] = RELEASED
        self._first_live = max(self._first_live, upto)

    def truncate(self, length: int) -> None:
        """Roll the committed history back to `length` (only within what is still held)."""
        if length < self._first_live * self.page_size and length < self.length:
            raise RuntimeError("KV cache: cannot roll back into pages the window has given back")
        self.length = min(self.length, length)
        self.pending = 0
        keep = max(self.pages_for(self.length), self._first_live)
        while len(self.pages) > keep:
            self.pool.release(self.pages.pop())

    def free(self) -> None:
        for i in range(self._first_live, len(self.pages)):
            self.pool.release(self.pages[i])
        self.pages = []
        self.length = self.pending = 0
        self._first_live = 0

    def slot_of(self, position: int) -> int:
        """Flat slot (page id * page_size + offset) of a position that is held."""
        page = self.pages[position // self.page_size]
        if page == RELEASED:
            raise RuntimeError(f"KV cache: position {position} lies in a page the window has given back")
        return page * self.page_size + position % self.page_size
