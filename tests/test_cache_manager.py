"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; slots."""
import random

import numpy as np
import pytest

from ginfer_b200.cache import NoFreeSlot, OutOfPages, PagePoolError
from ginfer_b200.cache.native import NativeCacheManager
from reference_cache import CacheManager as PyCacheManager
from reference_cache import PagePool, SlotPool


@pytest.fixture(params=["python", "native"])
def CacheManager(request):
    """Both managers: the one in Python that states the rules and the one in C++ that the engine
    runs (host code; it compiles and runs without a GPU)."""
    return PyCacheManager if request.param == "python" else NativeCacheManager


def test_pool_refuses_double_return_and_foreign_return():
    pool = PagePool(4)
    a = pool.take(2, owner=1)
    b = pool.take(2, owner=2)
    assert sorted(a + b) == [0, 1, 2, 3] and pool.num_free == 0
    with pytest.raises(OutOfPages):
        pool.take(1, owner=3)
    with pytest.raises(PagePoolError, match="held by"):
        pool.give_back([a[0]], owner=2)
    pool.give_back(a, owner=1)
    with pytest.raises(PagePoolError, match="twice"):
        pool.give_back([a[0]], owner=1)
    pool.check()
    assert pool.take(1, owner=5) == [a[-1]]          # the page given back last goes out first
    pool.check()


def test_slots():
    s = SlotPool(2)
    a, b = s.take("x"), s.take("y")
    assert {a, b} == {0, 1}
    with pytest.raises(NoFreeSlot):
        s.take("z")
    s.give_back(a)
    with pytest.raises(RuntimeError):
        s.give_back(a)
    assert s.take("z") == a and s.holder_of(a) == "z"


def test_reserve_commit_tables_and_slot_mapping(CacheManager):
    m = CacheManager([0], num_pages=6, page_size=4, max_num_seqs=2, max_seq_len=24)
    rc = m.admit("a")
    assert m.pages_needed("a", 5) == [2] and m.pages_needed("new", 9) == [3]
    m.reserve("a", 5)
    m.commit("a", 5)
    assert rc.num_tokens == 5 and m.free_pages() == [4]
    m.reserve("a", 3)                                 # 5..7 fit the second page
    assert m.free_pages() == [4]
    m.commit("a", 3)
    m.reserve("a", 1)                                 # token 8 opens a page
    assert m.free_pages() == [3]
    row = m.tables[0][rc.slot]
    assert (row[:3] >= 0).all() and (row[3:] == -1).all()
    pos = np.arange(9)
    sm = m.slot_mapping(0, np.full(9, rc.slot), pos)
    assert (sm == row[pos // 4] * 4 + pos % 4).all() and len(set(sm.tolist())) == 9
    m.check()
    with pytest.raises(ValueError, match="max_seq_len"):
        m.reserve("a", 16)
    m.release("a")
    assert m.free_pages() == [6] and not m.has("a")
    m.check()


def test_reserve_is_all_or_nothing_across_groups(CacheManager):
    m = CacheManager([0, 8], num_pages=[2, 8], page_size=4, max_num_seqs=2, max_seq_len=64)
    m.admit("a")
    with pytest.raises(OutOfPages):
        m.reserve("a", 12)                            # group 0 has 2 pages, 3 are needed
    assert m.free_pages() == [2, 8] and m.get("a").reserved == 0
    m.check()


def test_window_gives_pages_back_and_never_one_that_is_visible(CacheManager):
    P, W = 4, 10
    m = CacheManager([0, W], num_pages=40, page_size=P, max_num_seqs=1, max_seq_len=160)
    rc = m.admit("a")
    n = 0
    for step in [7, 1, 1, 13, 2, 1, 1, 1, 30, 1, 1, 5]:
        m.reserve("a", step)
        # everything the step's tokens see is in the table: position p sees (p - W, p]
        row = m.tables[1][rc.slot]
        for p in range(n, n + step):
            for c in range(max(0, p - W + 1), p + 1):
                assert row[c // P] >= 0, (p, c)
        m.commit("a", step)
        n += step
        m.check()
        first = rc.first_page[1]
        assert first == max(0, n - W + 1) // P       # dead pages are gone, and only those
        assert (m.tables[1][rc.slot][:first] == -1).all()
        assert rc.first_page[0] == 0                  # the full group keeps everything
    held = rc.next_page[1] - rc.first_page[1]
    assert held <= -(-W // P) + 1
    m.release("a")
    assert m.free_pages() == [40, 40]


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_page_accounted_for(CacheManager, seed):
    rng = random.Random(seed)
    P = rng.choice([1, 4, 16])
    windows = rng.choice([[0], [0, 24], [0, 7, 40]])
    pages = rng.choice([12, 30])
    m = CacheManager(windows, num_pages=pages, page_size=P, max_num_seqs=4,
                     max_seq_len=pages * P)
    live: dict[str, int] = {}
    issued = 0
    used_before: set[int] = set()
    reused = False
    for _ in range(400):
        act = rng.random()
        if act < 0.15 and len(live) < 4:
            rid = f"r{issued}"
            issued += 1
            m.admit(rid)
            live[rid] = 0
        elif act < 0.75 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 17])
            if live[rid] + n > m.max_seq_len:
                continue
            if m.can_reserve(rid, n):
                before = m.free_pages()
                need = m.pages_needed(rid, n)
                m.reserve(rid, n)
                assert m.free_pages() == [b - k for b, k in zip(before, need)]
                rc = m.get(rid)
                now = set(int(p) for p in
                          m.tables[0][rc.slot][rc.first_page[0]:rc.next_page[0]])
                reused |= bool(now & used_before)
                used_before |= now
                m.commit(rid, n)
                live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
        elif act < 0.85 and live:
            rid = rng.choice(list(live))
            m.release(rid, keep_slot=True)            # preempted: pages back, slot kept
            live[rid] = 0
            assert m.has(rid) and m.get(rid).num_tokens == 0
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.get(rid).num_tokens == n
    for rid in list(live):
        m.release(rid)
    m.check()
    assert m.free_pages() == [pages] * len(windows) and m.slots.num_free == 4
    assert reused, "the scenario never used a page again"


@pytest.mark.parametrize("seed", range(6))
def test_native_manager_does_what_the_python_manager_does(seed):
    """The same random sequence of operations on both managers: same answers, same tables, same
    free counts, same refusals, step by step; and the calls for a whole step agree with the calls
    per request."""
    rng = random.Random(100 + seed)
    P = rng.choice([1, 4, 16])
    windows = rng.choice([[0], [0, 24], [0, 7, 40]])
    pages = rng.choice([12, 30])
    a = PyCacheManager(windows, pages, P, 4, pages * P)
    b = NativeCacheManager(windows, pages, P, 4, pages * P)
    live: list[str] = []
    issued = 0

    def both(fn):
        out = []
        for m in (a, b):
            try:
                out.append(("ok", fn(m)))
            except (OutOfPages, ValueError, NoFreeSlot, KeyError) as e:
                out.append((type(e).__name__, None))
        assert out[0] == out[1], out
        return out[0]

    for _ in range(500):
        act = rng.random()
        if act < 0.15:
            rid = f"r{issued}"
            issued += 1
            if both(lambda m: m.admit(rid).slot)[0] == "ok":
                live.append(rid)
        elif act < 0.7 and live:
            rid, n = rng.choice(live), rng.choice([1, 1, 2, 5, 17, 40])
            both(lambda m: m.pages_needed(rid, n))
            both(lambda m: m.can_reserve(rid, n))
            if both(lambda m: m.reserve(rid, n))[0] == "ok":
                k = rng.randint(0, n)
                both(lambda m: m.commit(rid, k))
                both(lambda m: m.commit(rid, n - k))
        elif act < 0.8 and live:
            rid = rng.choice(live)
            both(lambda m: m.release(rid, keep_slot=True))
        elif act < 0.9 and live:
            rid = live.pop(rng.randrange(len(live)))
            both(lambda m: m.release(rid))
        elif live:
            # a whole step: need, then reserve, then commit, against the calls per request
            ids = rng.sample(live, rng.randint(1, len(live)))
            ns = [rng.choice([1, 1, 3, 9]) for _ in ids]
            slots = np.array([b.get(i).slot for i in ids])
            need, over = b.step_need(slots, np.array(ns))
            want = [sum(a.pages_needed(i, n)[g] for i, n in zip(ids, ns))
                    for g in range(len(windows))]
            assert need == want
            fits = all(a.get(i).num_tokens + a.get(i).reserved + n <= a.max_seq_len
                       for i, n in zip(ids, ns))
            assert (over < 0) == fits
            if fits and all(k <= f for k, f in zip(need, a.free_pages())):
                for i, n in zip(ids, ns):
                    a.reserve(i, n)
                b.reserve_step(slots, np.array(ns))
                assert list(b.lengths(slots)) == [a.get(i).num_tokens for i in ids]
                for i, n in zip(ids, ns):
                    a.commit(i, n)
                b.commit_step(slots, np.array(ns))
        a.check(), b.check()
        assert a.free_pages() == b.free_pages() and a.slots.num_free == b.slots.num_free
        for rid in live:
            ra, rb = a.get(rid), b.get(rid)
            assert (ra.slot, ra.num_tokens, ra.reserved, ra.first_page, ra.next_page) == \
                (rb.slot, rb.num_tokens, rb.reserved, rb.first_page, rb.next_page)
        for ta, tb in zip(a.tables, b.tables):
            assert (ta == tb).all()
