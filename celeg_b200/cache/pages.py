"""Host-side page accounting: a pool of page ids with reference counts.

Same contract as celeg's ``PagedBlockPool`` (src/runtime/concurrency/policy.cpp:21-111):
allocation is all-or-nothing, ``retain`` adds a reference, ``release`` validates every id
before it changes anything and throws on a page that is not held. Free pages are handed out
last-freed-first, so a page that was just given back is the next one used again.
"""
from __future__ import annotations

from typing import List, Optional, Sequence


class PageError(RuntimeError):
    """A page id is out of range, not held, or freed twice."""


class OutOfPages(RuntimeError):
    """The pool cannot serve an allocation; nothing was taken."""


class PagePool:
    def __init__(self, pages: int, page_tokens: int):
        if pages < 0 or page_tokens <= 0:
            raise ValueError("a page pool needs pages >= 0 and page_tokens > 0")
        self.page_tokens = page_tokens
        self._ref = [0] * pages
        self._free: List[int] = list(range(pages - 1, -1, -1))   # pop() yields 0, 1, 2, ...
        self.high_water = 0                                      # most pages ever out of the pool at once

    @property
    def total_pages(self) -> int:
        return len(self._ref)

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return len(self._ref) - len(self._free)

    def ref_count(self, page: int) -> int:
        self._check_id(page)
        return self._ref[page]

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_tokens - 1) // self.page_tokens

    def allocate(self, count: int) -> Optional[List[int]]:
        """``count`` pages with one reference each, or ``None`` if fewer are free."""
        if count < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if count > len(self._free):
            return None
        taken = [self._free.pop() for _ in range(count)]
        for page in taken:
            self._ref[page] = 1
        self.high_water = max(self.high_water, len(self._ref) - len(self._free))
        return taken

    def allocate_tokens(self, tokens: int) -> Optional[List[int]]:
        return self.allocate(self.pages_for(tokens))

    def retain(self, pages: Sequence[int]) -> None:
        for page in pages:
            self._check_id(page)
            if self._ref[page] == 0:
                raise PageError(f"page {page} is free and cannot be retained")
        for page in pages:
            self._ref[page] += 1

    def release(self, pages: Sequence[int]) -> None:
        drops = {}
        for page in pages:
            self._check_id(page)
            drops[page] = drops.get(page, 0) + 1
        for page, count in drops.items():
            if self._ref[page] < count:
                raise PageError(f"page {page} is released {count} time(s) but held {self._ref[page]} time(s)")
        for page in pages:
            self._ref[page] -= 1
            if self._ref[page] == 0:
                self._free.append(page)

    def _check_id(self, page: int) -> None:
        if not isinstance(page, int) or not 0 <= page < len(self._ref):
            raise PageError(f"page id {page!r} is outside the pool of {len(self._ref)} pages")
