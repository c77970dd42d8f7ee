"""What the cache manager raises."""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """The pool cannot give the pages asked for."""


class PagePoolError(RuntimeError):
    """A page was returned twice, returned by someone who does not hold it, or handed out while
    held."""


class NoFreeSlot(RuntimeError):
    """Every request slot is taken."""
