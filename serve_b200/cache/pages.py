"""A pool of cache pages: who holds which page, and which are free.

Host-side only. The reference keeps a Python list used as a stack
(serve/kv_cache_paged.py:29,59-60,73) and never checks for exhaustion; here
allocation either hands out all the pages asked for or raises ``OutOfPages``
and changes nothing, and a page is known to be either free or held by exactly
one owner.
"""
from __future__ import annotations

from typing import Dict, Hashable, List


class OutOfPages(RuntimeError):
    """The pool cannot hand out the pages asked for; nothing was taken."""

    def __init__(self, wanted: int, available: int, group: int = 0):
        super().__init__(f"cache group {group}: {wanted} pages wanted, {available} free")
        self.wanted = wanted
        self.available = available
        self.group = group


class PagePool:
    def __init__(self, num_pages: int, group: int = 0):
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self.group = group
        # stack: the page freed last is handed out first
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._owner: Dict[int, Hashable] = {}
        self.high_water = 0

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int, owner: Hashable) -> List[int]:
        if n < 0:
            raise ValueError("cannot take a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(n, len(self._free), self.group)
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._owner[p] = owner
        self.high_water = max(self.high_water, self.in_use)
        return pages

    def give_back(self, pages: List[int], owner: Hashable) -> None:
        for p in pages:
            if self._owner.get(p, _NOBODY) != owner:
                held = self._owner.get(p, _NOBODY)
                state = "free" if held is _NOBODY else f"held by {held!r}"
                raise RuntimeError(f"page {p} given back by {owner!r} but it is {state}")
        for p in pages:
            del self._owner[p]
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner.get(page)

    def check(self) -> None:
        """Every page is free or held, never both, never twice."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        held = set(self._owner)
        if free & held:
            raise AssertionError(f"pages both free and held: {sorted(free & held)}")
        if len(free) + len(held) != self.num_pages or (free | held) != set(range(self.num_pages)):
            raise AssertionError("a page was lost")


_NOBODY = object()
