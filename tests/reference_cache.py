"""The cache manager's rules in plain Python: the oracle that the tests compare the C++ manager
(``ginfer_b200/csrc/cache_core.cu`` behind ``ginfer_b200.cache.NativeCacheManager``, the one the
engine runs) with, operation by operation.  Not part of the product.

Reference: ``ginfer/engine/block_manager.{h,cc}``.  There one page id addresses all layers at
once, a prompt's pages are all taken at admission (``block_manager.cc:63-110``), decoding takes a
page when a token opens one (``:121-135``), and pages return when a request finishes or is
preempted (``ginfer/engine/scheduler.cc:73-77,92-94``).  Here

* layers with different needs form groups (all keys; the last ``window`` keys), each with a pool
  and block tables of its own;
* pages are taken for the tokens of one step at a time (:meth:`reserve`), so prompts can be fed
  in portions;
* a windowed group gives a page back as soon as no later token can see it (:meth:`commit`);
* each request also holds a slot for state of fixed size.


A pool of pages is a stack of free pages (the page given back last is handed out first; the
reference keeps a free deque and a used set and searches the deque on every allocation,
``ginfer/engine/block_manager.cc:41-61``) with an owner array that makes double hand-outs and
double returns errors.  A request takes a slot when it is admitted and keeps it until it ends,
also across a preemption that gives its pages back.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from ginfer_b200.cache.errors import NoFreeSlot, OutOfPages, PagePoolError


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


class SlotPool:
    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("at least one slot is needed")
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots - 1, -1, -1))
        self._holder: dict[int, object] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, holder) -> int:
        if not self._free:
            raise NoFreeSlot(f"all {self.num_slots} request slots are taken")
        s = self._free.pop()
        self._holder[s] = holder
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._holder:
            raise RuntimeError(f"slot {slot} is returned twice or was never taken")
        del self._holder[slot]
        self._free.append(slot)

    def holder_of(self, slot: int):
        return self._holder.get(slot)


@dataclass
class RequestCache:
    request_id: object
    slot: int
    owner: int                     # tag under which the pools know this request
    num_tokens: int = 0            # tokens whose keys are in the cache
    reserved: int = 0              # tokens beyond num_tokens that pages are taken for
    first_page: list[int] = field(default_factory=list)   # per group: lowest logical page held
    next_page: list[int] = field(default_factory=list)    # per group: first logical page not taken


class CacheManager:
    def __init__(self, group_windows: list[int], num_pages, page_size: int, max_num_seqs: int,
                 max_seq_len: int):
        """``group_windows[g]``: 0 if group ``g`` keeps all keys, else its window.
        ``num_pages``: pages per group (an int for all groups alike, or one per group)."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = int(page_size)
        self.windows = [int(w) for w in group_windows]
        n = len(self.windows)
        counts = [int(num_pages)] * n if np.isscalar(num_pages) else [int(x) for x in num_pages]
        if len(counts) != n:
            raise ValueError("one page count per group is needed")
        self.pools = [PagePool(c) for c in counts]
        self.slots = SlotPool(max_num_seqs)
        self.max_seq_len = int(max_seq_len)
        self.table_width = -(-self.max_seq_len // self.page_size)
        # block tables by slot: tables[g][slot, logical page] = physical page or -1
        self.tables = [np.full((max_num_seqs, self.table_width), -1, dtype=np.int32)
                       for _ in range(n)]
        self.requests: dict[object, RequestCache] = {}
        self._next_owner = 0

    # ------------------------------------------------------------------ admission and release
    @property
    def num_groups(self) -> int:
        return len(self.pools)

    def has(self, request_id) -> bool:
        return request_id in self.requests

    def get(self, request_id) -> RequestCache:
        return self.requests[request_id]

    def admit(self, request_id) -> RequestCache:
        """Give the request a slot (no pages yet)."""
        if request_id in self.requests:
            raise KeyError(f"request {request_id!r} is live already")
        slot = self.slots.take(request_id)
        rc = RequestCache(request_id, slot, self._next_owner,
                          first_page=[0] * self.num_groups, next_page=[0] * self.num_groups)
        self._next_owner += 1
        self.requests[request_id] = rc
        return rc

    def release(self, request_id, keep_slot: bool = False) -> None:
        """Give back every page of the request; with ``keep_slot`` it stays admitted with nothing
        cached (a preempted request that will be computed again)."""
        rc = self.requests[request_id]
        for g, pool in enumerate(self.pools):
            row = self.tables[g][rc.slot]
            held = row[rc.first_page[g]:rc.next_page[g]]
            pool.give_back([int(p) for p in held if p >= 0], rc.owner)
            row[:rc.next_page[g]] = -1
            rc.first_page[g] = rc.next_page[g] = 0
        rc.num_tokens = rc.reserved = 0
        if not keep_slot:
            self.slots.give_back(rc.slot)
            del self.requests[request_id]

    # ------------------------------------------------------------------ pages for a step
    def _new_pages(self, next_page: int, have_tokens: int, n_new: int) -> int:
        end_page = -(-(have_tokens + n_new) // self.page_size)
        return max(0, end_page - next_page)

    def pages_needed(self, request_id, n_new: int) -> list[int]:
        """Pages per group that :meth:`reserve` would take for ``n_new`` more tokens."""
        rc = self.requests.get(request_id)
        if rc is None:
            return [-(-n_new // self.page_size)] * len(self.pools)
        end_page = -(-(rc.num_tokens + rc.reserved + n_new) // self.page_size)
        return [end_page - p if end_page > p else 0 for p in rc.next_page]

    def free_pages(self) -> list[int]:
        return [p.num_free for p in self.pools]

    def can_reserve(self, request_id, n_new: int, already: list[int] | None = None) -> bool:
        """``already``: pages per group that the caller has promised to others in this step."""
        need = self.pages_needed(request_id, n_new)
        if not any(need):
            return True
        free = self.free_pages()
        if already is not None:
            free = [f - a for f, a in zip(free, already)]
        return all(n <= f for n, f in zip(need, free))

    def reserve(self, request_id, n_new: int) -> None:
        """Take pages so that the next ``n_new`` tokens of the request have slots, in every group
        or (if one pool is short) in none."""
        rc = self.requests[request_id]
        have = rc.num_tokens + rc.reserved
        if have + n_new > self.max_seq_len:
            raise ValueError(f"request {request_id!r} would hold {have + n_new} tokens; "
                             f"max_seq_len is {self.max_seq_len}")
        need = [self._new_pages(rc.next_page[g], have, n_new) for g in range(self.num_groups)]
        for g, pool in enumerate(self.pools):
            if need[g] > pool.num_free:
                raise OutOfPages(f"group {g}: request {request_id!r} needs {need[g]} pages for "
                                 f"{n_new} tokens, {pool.num_free} are free")
        for g, pool in enumerate(self.pools):
            if need[g]:
                pages = pool.take(need[g], rc.owner)
                a = rc.next_page[g]
                self.tables[g][rc.slot, a:a + need[g]] = pages
                rc.next_page[g] = a + need[g]
        rc.reserved += n_new

    def commit(self, request_id, n: int) -> None:
        """``n`` reserved tokens are now in the cache.  Windowed groups give back the pages no
        later token can see: a token at position ``p >= num_tokens`` sees keys ``> p - window``,
        so a page whose last position is ``<= num_tokens - window`` is dead."""
        rc = self.requests[request_id]
        if n > rc.reserved:
            raise ValueError(f"commit of {n} tokens but only {rc.reserved} are reserved")
        rc.reserved -= n
        rc.num_tokens += n
        for g, w in enumerate(self.windows):
            if w <= 0:
                continue
            dead_end = max(0, rc.num_tokens - w + 1) // self.page_size    # pages [first, dead_end)
            dead_end = min(dead_end, rc.next_page[g])
            if dead_end > rc.first_page[g]:
                row = self.tables[g][rc.slot]
                self.pools[g].give_back([int(p) for p in row[rc.first_page[g]:dead_end]],
                                        rc.owner)
                row[rc.first_page[g]:dead_end] = -1
                rc.first_page[g] = dead_end

    # ------------------------------------------------------------------ what the step needs
    def slot_mapping(self, group: int, slots_of_token: np.ndarray, positions: np.ndarray
                     ) -> np.ndarray:
        """Physical token slot of each (request slot, position)."""
        pages = self.tables[group][slots_of_token, positions // self.page_size]
        return pages * self.page_size + positions % self.page_size

    def block_table(self, group: int, slot_ids: np.ndarray, width: int) -> np.ndarray:
        return self.tables[group][slot_ids, :width]

    # ------------------------------------------------------------------ checks
    def check(self) -> None:
        """No page lost, held twice, or in a table without being held by that request."""
        for g, pool in enumerate(self.pools):
            pool.check()
            seen: dict[int, object] = {}
            for rc in self.requests.values():
                row = self.tables[g][rc.slot]
                live = [int(p) for p in row[rc.first_page[g]:rc.next_page[g]]]
                if any(p < 0 for p in live):
                    raise AssertionError(f"request {rc.request_id!r} has a hole in group {g}")
                if (row[:rc.first_page[g]] >= 0).any() or (row[rc.next_page[g]:] >= 0).any():
                    raise AssertionError(f"request {rc.request_id!r} lists pages it gave back")
                for p in live:
                    if p in seen:
                        raise AssertionError(f"page {p} of group {g} is in the tables of "
                                             f"{seen[p]!r} and {rc.request_id!r}")
                    seen[p] = rc.request_id
                    if pool.owner_of(p) != rc.owner:
                        raise AssertionError(f"page {p} of group {g} is listed by "
                                             f"{rc.request_id!r} but held by another")
                if sorted(live) != sorted(pool.held_by(rc.owner)):
                    raise AssertionError(f"request {rc.request_id!r} holds pages of group {g} "
                                         "that its table does not list")
            if len(seen) + pool.num_free != pool.num_pages:
                raise AssertionError(f"group {g}: {pool.num_pages - pool.num_free - len(seen)} "
                                     "pages are held by no live request")
