"""A pool of cache pages: which are free, who holds the others.

The reference keeps a free deque and a used set and searches the deque on every allocation
(``ginfer/engine/block_manager.cc:41-61``).  Here the free pages are a stack (the page given back
last is handed out first) and an owner array makes double hand-outs and double returns errors
instead of silent corruption.
"""
from __future__ import annotations

import numpy as np


class OutOfPages(RuntimeError):
    """The pool cannot give the pages asked for."""


class PagePoolError(RuntimeError):
    """A page was returned twice, returned by someone who does not hold it, or handed out while
    held."""


class PagePool:
    FREE = -1

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))       # pop() gives page 0 first
        self._owner = np.full(self.num_pages, self.FREE, dtype=np.int64)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, n: int, owner: int) -> list[int]:
        if owner < 0:
            raise ValueError("owner ids are non-negative")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages asked, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._owner[p] != self.FREE:
                raise PagePoolError(f"page {p} was on the free list while held by "
                                    f"{self._owner[p]}")
            self._owner[p] = owner
        return out

    def give_back(self, pages, owner: int) -> None:
        for p in pages:
            p = int(p)
            if not (0 <= p < self.num_pages):
                raise PagePoolError(f"page {p} is not of this pool")
            if self._owner[p] == self.FREE:
                raise PagePoolError(f"page {p} is returned twice")
            if self._owner[p] != owner:
                raise PagePoolError(f"page {p} is held by {self._owner[p]}, not by {owner}")
            self._owner[p] = self.FREE
            self._free.append(p)

    def owner_of(self, page: int) -> int:
        return int(self._owner[page])

    def held_by(self, owner: int) -> list[int]:
        return [int(p) for p in np.nonzero(self._owner == owner)[0]]

    def check(self) -> None:
        """Every page is either free once or held once."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise PagePoolError("a page is on the free list twice")
        held = set(int(p) for p in np.nonzero(self._owner != self.FREE)[0])
        if held & set(free):
            raise PagePoolError(f"pages both free and held: {sorted(held & set(free))}")
        if len(held) + len(free) != self.num_pages:
            lost = set(range(self.num_pages)) - held - set(free)
            raise PagePoolError(f"pages lost: {sorted(lost)}")
