"""The cache manager: :class:`NativeCacheManager` keeps pools, slots, block tables and the
reserve/commit/release rules in C++ (``csrc/cache_core.cu``, host code only).

Reference: ``ginfer/engine/block_manager.{h,cc}``.  There one page id addresses all layers at
once, a prompt's pages are all taken at admission (``block_manager.cc:63-110``), decoding takes a
page when a token opens one (``:121-135``), and pages return when a request finishes or is
preempted (``ginfer/engine/scheduler.cc:73-77,92-94``).  Here

* layers with different needs form groups (all keys; the last ``window`` keys), each with a pool
  (a stack of free pages and an owner array: a page handed out twice, returned twice or returned
  by a stranger is an error) and block tables of its own;
* pages are taken for the tokens of one step at a time (``reserve``), in every group or in none,
  so prompts can be fed in portions;
* a windowed group gives a page back as soon as no later token can see it (``commit``: a page is
  dead once its last position is ``<= len - window``);
* each request also holds a slot for state of fixed size, from admission until it ends (also
  across a preemption that gives its pages back); ``check()`` proves that no page is lost, held
  twice or listed without being held.

The tests hold every operation against the same rules written in plain Python.

The block tables are numpy arrays owned here and written by the C++ side, so the step function
gathers slot mappings and table rows from them as before.  Besides the per-request calls there are
calls for a whole step (:meth:`step_need`, :meth:`reserve_step`, :meth:`commit_step`): one crossing
into native code per step instead of several per request.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p

import numpy as np

from .errors import NoFreeSlot, OutOfPages, PagePoolError

_OK, _OUT_OF_PAGES, _POOL_ERROR, _NO_FREE_SLOT, _BAD_VALUE, _NOT_LIVE, _CHECK_FAILED = range(7)


def _lib():
    from ..ops.build import load_library
    lib = load_library("cache_core")
    if not getattr(lib, "_gf_typed", False):
        ip = POINTER(c_int)
        lib.gf_cm_create.restype = c_void_p
        lib.gf_cm_create.argtypes = [c_int, ip, ip, c_int, c_int, c_int, POINTER(c_void_p)]
        lib.gf_cm_destroy.restype = None
        lib.gf_cm_destroy.argtypes = [c_void_p]
        lib.gf_cm_error.restype = c_char_p
        lib.gf_cm_error.argtypes = [c_void_p]
        lib.gf_cm_table_width.argtypes = [c_void_p]
        lib.gf_cm_free_slots.argtypes = [c_void_p]
        lib.gf_cm_free_pages.restype = None
        lib.gf_cm_free_pages.argtypes = [c_void_p, ip]
        lib.gf_cm_admit.argtypes = [c_void_p, ip]
        lib.gf_cm_get.argtypes = [c_void_p, c_int, POINTER(c_longlong)]
        lib.gf_cm_pages_needed.argtypes = [c_void_p, c_int, c_int, ip]
        lib.gf_cm_lengths.argtypes = [c_void_p, ip, c_int, ip]
        lib.gf_cm_step_need.argtypes = [c_void_p, ip, ip, c_int, ip, ip]
        lib.gf_cm_reserve.argtypes = [c_void_p, c_int, c_int]
        lib.gf_cm_commit.argtypes = [c_void_p, c_int, c_int]
        lib.gf_cm_reserve_many.argtypes = [c_void_p, ip, ip, c_int]
        lib.gf_cm_commit_many.argtypes = [c_void_p, ip, ip, c_int]
        lib.gf_cm_release.argtypes = [c_void_p, c_int, c_int]
        lib.gf_cm_check.argtypes = [c_void_p]
        lib.gf_sched_decide.argtypes = [c_void_p, c_int, c_int, c_int, c_int] + [ip] * 9
        lib._gf_typed = True
    return lib


class _Request:
    """A live request's record; the numbers are read from the native side when asked for."""

    def __init__(self, manager: "NativeCacheManager", request_id, slot: int):
        self._m, self.request_id, self.slot = manager, request_id, slot

    def _read(self):
        return self._m._get(self.slot)

    @property
    def num_tokens(self) -> int:
        return self._read()[0]

    @property
    def reserved(self) -> int:
        return self._read()[1]

    @property
    def owner(self) -> int:
        return self._read()[2]

    @property
    def first_page(self) -> list[int]:
        g = self._m.num_groups
        return self._read()[3:3 + g]

    @property
    def next_page(self) -> list[int]:
        g = self._m.num_groups
        return self._read()[3 + g:3 + 2 * g]


class _Slots:
    def __init__(self, manager: "NativeCacheManager"):
        self._m = manager
        self.num_slots = manager.max_num_seqs

    @property
    def num_free(self) -> int:
        return int(self._m._lib.gf_cm_free_slots(self._m._h))

    def holder_of(self, slot: int):
        for rid, rc in self._m.requests.items():
            if rc.slot == slot:
                return rid
        return None


class _Pool:
    def __init__(self, manager: "NativeCacheManager", group: int):
        self._m, self._g = manager, group
        self.num_pages = manager.num_pages[group]

    @property
    def num_free(self) -> int:
        return self._m.free_pages()[self._g]


class NativeCacheManager:
    def __init__(self, group_windows: list[int], num_pages, page_size: int, max_num_seqs: int,
                 max_seq_len: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self._lib = _lib()
        self.page_size = int(page_size)
        self.windows = [int(w) for w in group_windows]
        n = len(self.windows)
        counts = [int(num_pages)] * n if np.isscalar(num_pages) else [int(x) for x in num_pages]
        if len(counts) != n:
            raise ValueError("one page count per group is needed")
        if any(c <= 0 for c in counts):
            raise ValueError("a page pool needs at least one page")
        if max_num_seqs <= 0:
            raise ValueError("at least one slot is needed")
        self.num_pages = counts
        self.max_num_seqs = int(max_num_seqs)
        self.max_seq_len = int(max_seq_len)
        self.table_width = -(-self.max_seq_len // self.page_size)
        self.tables = [np.full((self.max_num_seqs, self.table_width), -1, dtype=np.int32)
                       for _ in range(n)]
        ptrs = (c_void_p * n)(*[t.ctypes.data for t in self.tables])
        self._h = self._lib.gf_cm_create(n, (c_int * n)(*counts), (c_int * n)(*self.windows),
                                         self.page_size, self.max_num_seqs, self.max_seq_len, ptrs)
        if not self._h:
            raise ValueError("the cache manager refused its sizes")
        self.requests: dict[object, _Request] = {}
        self.slots = _Slots(self)
        self.pools = [_Pool(self, g) for g in range(n)]
        self._ints = (c_int * max(8, n))()
        self._rec = (c_longlong * (3 + 2 * n))()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.gf_cm_destroy(h)

    # ------------------------------------------------------------------ errors
    def _raise(self, code: int):
        msg = self._lib.gf_cm_error(self._h).decode()
        if code == _OUT_OF_PAGES:
            raise OutOfPages(msg)
        if code == _POOL_ERROR:
            raise PagePoolError(msg)
        if code == _NO_FREE_SLOT:
            raise NoFreeSlot(msg)
        if code == _BAD_VALUE:
            raise ValueError(msg)
        if code == _NOT_LIVE:
            raise KeyError(msg)
        raise AssertionError(msg)

    def _get(self, slot: int) -> list[int]:
        rc = self._lib.gf_cm_get(self._h, slot, self._rec)
        if rc:
            self._raise(rc)
        return [int(v) for v in self._rec]

    # ------------------------------------------------------------------ admission and release
    @property
    def num_groups(self) -> int:
        return len(self.windows)

    def has(self, request_id) -> bool:
        return request_id in self.requests

    def get(self, request_id) -> _Request:
        return self.requests[request_id]

    def admit(self, request_id) -> _Request:
        if request_id in self.requests:
            raise KeyError(f"request {request_id!r} is live already")
        slot = c_int(-1)
        rc = self._lib.gf_cm_admit(self._h, ctypes.byref(slot))
        if rc:
            self._raise(rc)
        r = _Request(self, request_id, slot.value)
        self.requests[request_id] = r
        return r

    def release(self, request_id, keep_slot: bool = False) -> None:
        r = self.requests[request_id]
        rc = self._lib.gf_cm_release(self._h, r.slot, int(bool(keep_slot)))
        if rc:
            self._raise(rc)
        if not keep_slot:
            del self.requests[request_id]

    # ------------------------------------------------------------------ pages for a step
    def pages_needed(self, request_id, n_new: int) -> list[int]:
        r = self.requests.get(request_id)
        rc = self._lib.gf_cm_pages_needed(self._h, -1 if r is None else r.slot, int(n_new),
                                          self._ints)
        if rc:
            self._raise(rc)
        return [int(self._ints[g]) for g in range(self.num_groups)]

    def free_pages(self) -> list[int]:
        self._lib.gf_cm_free_pages(self._h, self._ints)
        return [int(self._ints[g]) for g in range(self.num_groups)]

    def can_reserve(self, request_id, n_new: int, already: list[int] | None = None) -> bool:
        need = self.pages_needed(request_id, n_new)
        if not any(need):
            return True
        free = self.free_pages()
        if already is not None:
            free = [f - a for f, a in zip(free, already)]
        return all(k <= f for k, f in zip(need, free))

    def reserve(self, request_id, n_new: int) -> None:
        rc = self._lib.gf_cm_reserve(self._h, self.requests[request_id].slot, int(n_new))
        if rc:
            if rc == _BAD_VALUE:
                raise ValueError(f"request {request_id!r}: "
                                 f"{self._lib.gf_cm_error(self._h).decode()} (max_seq_len)")
            self._raise(rc)

    def commit(self, request_id, n: int) -> None:
        rc = self._lib.gf_cm_commit(self._h, self.requests[request_id].slot, int(n))
        if rc:
            self._raise(rc)

    # ------------------------------------------------------------------ a whole step at once
    def step_need(self, slots: np.ndarray, n_new: np.ndarray) -> tuple[list[int], int]:
        """Pages per group that the step's entries need together (``slots[i] < 0``: a request not
        admitted yet) and the index of the first entry that would pass ``max_seq_len`` (-1: none)."""
        slots = np.ascontiguousarray(slots, dtype=np.int32)
        n_new = np.ascontiguousarray(n_new, dtype=np.int32)
        over = c_int(-1)
        ip = POINTER(c_int)
        rc = self._lib.gf_cm_step_need(self._h, slots.ctypes.data_as(ip), n_new.ctypes.data_as(ip),
                                       int(slots.size), self._ints, ctypes.byref(over))
        if rc:
            self._raise(rc)
        return [int(self._ints[g]) for g in range(self.num_groups)], over.value

    def lengths(self, slots: np.ndarray) -> np.ndarray:
        """Tokens in the cache of the requests that hold ``slots``."""
        slots = np.ascontiguousarray(slots, dtype=np.int32)
        out = np.empty(slots.size, dtype=np.int32)
        ip = POINTER(c_int)
        rc = self._lib.gf_cm_lengths(self._h, slots.ctypes.data_as(ip), int(slots.size),
                                     out.ctypes.data_as(ip))
        if rc:
            self._raise(rc)
        return out

    def reserve_step(self, slots: np.ndarray, n_new: np.ndarray) -> None:
        slots = np.ascontiguousarray(slots, dtype=np.int32)
        n_new = np.ascontiguousarray(n_new, dtype=np.int32)
        ip = POINTER(c_int)
        rc = self._lib.gf_cm_reserve_many(self._h, slots.ctypes.data_as(ip),
                                          n_new.ctypes.data_as(ip), int(slots.size))
        if rc:
            self._raise(rc)

    def commit_step(self, slots: np.ndarray, n: np.ndarray) -> None:
        slots = np.ascontiguousarray(slots, dtype=np.int32)
        n = np.ascontiguousarray(n, dtype=np.int32)
        ip = POINTER(c_int)
        rc = self._lib.gf_cm_commit_many(self._h, slots.ctypes.data_as(ip), n.ctypes.data_as(ip),
                                         int(slots.size))
        if rc:
            self._raise(rc)

    # ------------------------------------------------------------------ the scheduler's decision
    def decide(self, budget: int, max_num_seqs: int, running: list, waiting: list):
        """One scheduling decision in native code (``gf_sched_decide`` in ``csrc/cache_core.cu``;
        the rules are those of ``engine/scheduler.py``).  ``running`` and ``waiting``: lists of
        ``(request_id, tokens, computed)`` in order.  Pages of preempted requests are released and
        admitted requests get their slots here.  Returns ``(batch, running_order, waiting_order,
        preempts, dropped)``: ``batch`` = ``(entry, start, n, sample)`` tuples with entries
        numbered through ``running + waiting``; the orders are entry numbers; ``preempts[e]`` says
        how often entry ``e`` was preempted, ``dropped[e]`` whether it was given up."""
        reqs = list(running) + list(waiting)
        n, nr = len(reqs), len(running)
        slot = np.fromiter((self.requests[r[0]].slot if r[0] in self.requests else -1
                            for r in reqs), dtype=np.int32, count=n)
        slot_in = slot.copy()
        tokens = np.fromiter((r[1] for r in reqs), dtype=np.int32, count=n)
        computed = np.fromiter((r[2] for r in reqs), dtype=np.int32, count=n)
        preempts = np.zeros(n, dtype=np.int32)
        dropped = np.zeros(n, dtype=np.int32)
        batch = np.zeros(4 * max(n, 1), dtype=np.int32)
        order = np.zeros(max(n, 1), dtype=np.int32)
        n_batch, n_running = c_int(0), c_int(0)
        ip = POINTER(c_int)
        rc = self._lib.gf_sched_decide(
            self._h, int(budget), int(max_num_seqs), nr, n - nr, slot.ctypes.data_as(ip),
            tokens.ctypes.data_as(ip), computed.ctypes.data_as(ip), preempts.ctypes.data_as(ip),
            dropped.ctypes.data_as(ip), batch.ctypes.data_as(ip), ctypes.byref(n_batch),
            order.ctypes.data_as(ip), ctypes.byref(n_running))
        if rc:
            self._raise(rc)
        for e in range(n):                         # slots taken and given back on the native side
            rid = reqs[e][0]
            if slot_in[e] < 0 <= slot[e]:
                self.requests[rid] = _Request(self, rid, int(slot[e]))
            elif slot_in[e] >= 0 > slot[e]:
                del self.requests[rid]
        acts = [tuple(int(v) for v in batch[4 * i:4 * i + 4]) for i in range(n_batch.value)]
        k = n_running.value
        live = n - int(dropped.sum())
        return (acts, [int(e) for e in order[:k]], [int(e) for e in order[k:live]],
                preempts.tolist(), dropped.tolist())

    # ------------------------------------------------------------------ what the step needs
    def slot_mapping(self, group: int, slots_of_token: np.ndarray, positions: np.ndarray
                     ) -> np.ndarray:
        pages = self.tables[group][slots_of_token, positions // self.page_size]
        return pages * self.page_size + positions % self.page_size

    def block_table(self, group: int, slot_ids: np.ndarray, width: int) -> np.ndarray:
        return self.tables[group][slot_ids, :width]

    # ------------------------------------------------------------------ checks
    def check(self) -> None:
        rc = self._lib.gf_cm_check(self._h)
        if rc:
            raise AssertionError(self._lib.gf_cm_error(self._h).decode())
        live = {r.slot for r in self.requests.values()}
        if len(live) != len(self.requests) or \
                len(live) + self.slots.num_free != self.max_num_seqs:
            raise AssertionError("the slots of the live requests and the free slots do not add up")
