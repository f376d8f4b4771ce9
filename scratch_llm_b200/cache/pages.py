"""Host-side accounting of one group's pages: which are free, which are held, by whom.

The reference's paged cache keeps a free list and per-block reference counts
(src/scratch_llm/kv_cache.py:330-359) and raises when the pool is exhausted (:341-345).  Here
an allocation that cannot be met returns None, so running out of pages is a decision of the
scheduler and never an exception in the middle of a step.  Pages come back last-in first-out,
so a small pool provably hands a freed page out again.
"""

from __future__ import annotations


class PageAccountingError(AssertionError):
    """A page was freed twice, freed by someone who does not hold it, or handed out while
    held: a fault of the cache manager, never of the caller's input."""


class PagePool:
    def __init__(self, n_pages: int) -> None:
        if n_pages < 1:
            raise ValueError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free: list[int] = list(range(n_pages - 1, -1, -1))  # pop() hands out page 0 first
        self._holder: dict[int, object] = {}

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._holder)

    def alloc(self, n: int, holder: object) -> list[int] | None:
        """``n`` pages for ``holder``, or None (and nothing taken) if fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            if p in self._holder:
                raise PageAccountingError(f"page {p} handed out while held by "
                                          f"{self._holder[p]!r}")
            self._holder[p] = holder
        return pages

    def free(self, pages: list[int], holder: object) -> None:
        for p in pages:
            if self._holder.get(p, _NOBODY) != holder:
                raise PageAccountingError(
                    f"page {p} freed by {holder!r} but held by "
                    f"{self._holder.get(p, 'nobody (double free)')!r}")
            del self._holder[p]
            self._free.append(p)

    def holder_of(self, page: int) -> object | None:
        return self._holder.get(page)

    def check(self) -> None:
        """Every page is free or held, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageAccountingError("a page is on the free list twice")
        if free & set(self._holder):
            raise PageAccountingError("a page is both free and held")
        if len(free) + len(self._holder) != self.n_pages:
            raise PageAccountingError(f"{self.n_pages - len(free) - len(self._holder)} pages "
                                      "are neither free nor held")


_NOBODY = object()
