"""A pool of fixed-size cache pages: the host-side allocator.

Pages are plain integers.  The pool knows which are free and which are held;
giving back a page that is not held, or asking for more than there are, is an
error, never a silent repair.
"""
from __future__ import annotations


class CacheError(RuntimeError):
    pass


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise CacheError(f"a pool cannot have {n_pages} pages")
        self.n_pages = n_pages
        # lowest page numbers are handed out first; freed pages are reused first
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def take(self, n: int) -> list[int]:
        if n < 0:
            raise CacheError(f"cannot take {n} pages")
        if n > len(self._free):
            raise CacheError(f"cache is full: {n} page(s) wanted, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages) -> None:
        pages = list(pages)
        for p in pages:
            if not (0 <= p < self.n_pages):
                raise CacheError(f"page {p} does not belong to this pool of {self.n_pages}")
            if not self._held[p]:
                raise CacheError(f"page {p} is given back twice (or was never taken)")
            self._held[p] = False
        self._free.extend(reversed(pages))

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is in the free list twice")
        for p in range(self.n_pages):
            if self._held[p] == (p in free):
                raise CacheError(f"page {p} is {'both held and free' if self._held[p] else 'lost'}")
