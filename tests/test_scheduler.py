"""The scheduler's decisions on the host, with the cache manager and a stand-in for the model."""
import random

import pytest

from ginfer_b200.cache.native import NativeCacheManager
from ginfer_b200.engine.request import Request, RequestState
from ginfer_b200.engine.scheduler import Scheduler
from ginfer_b200.sampling import SamplingParams, uniform
from reference_cache import CacheManager as PyCacheManager
from reference_scheduler import PythonScheduler


_MANAGER = [NativeCacheManager]


@pytest.fixture(autouse=True, params=["native", "python"])
def _both_managers(request):
    """Every test here runs over the C++ cache manager (what the engine uses) and the Python one."""
    _MANAGER[0] = NativeCacheManager if request.param == "native" else PyCacheManager
    yield


def _sched(pages=16, page=4, seqs=4, budget=16, max_len=64, eos=(), windows=(0,)):
    cache = _MANAGER[0](list(windows), pages, page, seqs, max_len)
    # the engine's scheduler (decision in C++) over the engine's manager; the same rules in
    # plain Python over the plain-Python manager
    cls = Scheduler if _MANAGER[0] is NativeCacheManager else PythonScheduler
    return cls(cache, seqs, budget, max_len, eos), cache


def _next_token(req):
    """A stand-in model: the next token is a function of the tokens so far (so a request that is
    computed again after a preemption must get the same continuation)."""
    h = 17
    for i in range(req.num_tokens):
        h = (h * 31 + req.token_at(i)) % 1009
    return h % 97


def _run_step(sched, cache, log=None):
    batch, dropped = sched.schedule()
    for s in batch:                                   # what the runner does with the pages
        assert s.start == cache.get(s.request.request_id).num_tokens == s.request.num_computed
        cache.reserve(s.request.request_id, s.num_tokens)
    for s in batch:
        cache.commit(s.request.request_id, s.num_tokens)
    tokens = []
    for s in batch:
        if s.sample:
            assert s.start + s.num_tokens == s.request.num_tokens
            tokens.append(_next_token(s.request))
    if log is not None:
        log.append([(s.request.request_id, s.start, s.num_tokens, s.sample) for s in batch])
    finished = sched.postprocess(batch, tokens)
    cache.check()
    return batch, dropped + finished


def _req(i, n, max_tokens=4, **kw):
    return Request(i, [(7 * i + j) % 50 for j in range(n)],
                   SamplingParams(max_tokens=max_tokens, **kw))


def test_prompt_is_cut_under_the_budget_and_decode_goes_first():
    sched, cache = _sched(pages=32, budget=10)
    a, b = _req(0, 23, max_tokens=3), _req(1, 4, max_tokens=6)
    sched.add(a)
    sched.add(b)
    log = []
    _run_step(sched, cache, log)
    assert log[-1] == [(0, 0, 10, False)]            # b waits: the budget is spent
    _run_step(sched, cache, log)
    assert log[-1] == [(0, 10, 10, False)]
    _run_step(sched, cache, log)
    assert log[-1] == [(0, 20, 3, True), (1, 0, 4, True)]
    _run_step(sched, cache, log)
    assert log[-1] == [(0, 23, 1, True), (1, 4, 1, True)]      # both decode
    while not sched.is_finished():
        batch, _ = _run_step(sched, cache, log)
        assert sum(n for _, _, n, _ in log[-1]) <= 10
    assert len(a.output) == 3 and len(b.output) == 6
    assert a.finish_reason == b.finish_reason == "max_tokens"
    assert cache.free_pages() == [32] and cache.slots.num_free == 4


def test_decode_tokens_come_before_prompt_portions():
    sched, cache = _sched(pages=64, budget=8, max_len=128)
    a = _req(0, 3, max_tokens=10)
    sched.add(a)
    _run_step(sched, cache)
    b = _req(1, 30, max_tokens=2)
    sched.add(b)
    log = []
    _run_step(sched, cache, log)
    assert log[-1] == [(0, 3, 1, True), (1, 0, 7, False)]      # one decode token, then 7 of b


def test_eos_finishes_unless_ignored_and_max_seq_len_stops():
    sched, cache = _sched(eos=(_next_token(_req(0, 5)),))
    a = _req(0, 5, max_tokens=9)
    b = _req(1, 5, max_tokens=9, ignore_eos=True)
    b.prompt = list(a.prompt)
    sched.add(a)
    sched.add(b)
    while not sched.is_finished():
        _run_step(sched, cache)
    assert a.finish_reason == "eos" and len(a.output) == 1
    assert b.finish_reason == "max_tokens" and len(b.output) == 9
    sched, cache = _sched(max_len=8, pages=8)
    c = _req(2, 6, max_tokens=50)
    sched.add(c)
    while not sched.is_finished():
        _run_step(sched, cache)
    assert c.finish_reason == "max_seq_len" and c.num_tokens == 8


def test_prompts_that_can_never_fit_are_refused_when_added():
    sched, _ = _sched(pages=4, page=4, max_len=64)
    with pytest.raises(ValueError, match="pages"):
        sched.add(_req(0, 17))
    with pytest.raises(ValueError, match="max_seq_len"):
        sched.add(_req(1, 64))
    with pytest.raises(ValueError, match="at least one"):
        sched.add(_req(2, 0))


def test_out_of_pages_preempts_the_youngest_which_is_computed_again():
    # 6 pages of 4 tokens; two requests of 9 tokens take 3 pages each; the first to need a
    # fourth page takes it from the younger one
    sched, cache = _sched(pages=6, page=4, budget=32, max_len=24)
    a, b = _req(0, 9, max_tokens=8), _req(1, 9, max_tokens=8)
    ref = []
    for r in (_req(0, 9, max_tokens=8), _req(1, 9, max_tokens=8)):    # each alone
        s2, c2 = _sched(pages=6, page=4, budget=32, max_len=24)
        s2.add(r)
        while not s2.is_finished():
            _run_step(s2, c2)
        ref.append(list(r.output))
    sched.add(a)
    sched.add(b)
    steps = 0
    while not sched.is_finished():
        _run_step(sched, cache)
        steps += 1
        assert steps < 200
    assert sched.num_preemptions >= 1 and b.num_preemptions >= 1 and a.num_preemptions == 0
    assert [a.output, b.output] == ref                # preemption does not change the result
    assert a.finish_reason == b.finish_reason == "max_tokens"
    assert cache.free_pages() == [6] and cache.slots.num_free == 4


class _PipelinedHost:
    """Drives a scheduler in the order of ``Engine.step`` with ``pipeline=True``: the step in
    flight is advanced, the following step is scheduled, prepared and launched (pages reserved
    and committed), and only then are the tokens of the step in flight resolved."""

    def __init__(self, sched, cache):
        self.sched, self.cache, self.flight = sched, cache, None
        self.returned = []

    def _launch(self, batch):
        for s in batch:
            assert s.start == self.cache.get(s.request.request_id).num_tokens
            self.cache.reserve(s.request.request_id, s.num_tokens)
        for s in batch:
            self.cache.commit(s.request.request_id, s.num_tokens)
        return batch

    @staticmethod
    def _tokens(batch):
        """What the stand-in model answers: a function of the request's known tokens (its
        placeholder for the token being chosen left out)."""
        out = []
        for s in batch:
            if s.sample:
                r = s.request
                known = (r.prompt + r.output)[:s.start + s.num_tokens]
                h = 17
                for t in known:
                    h = (h * 31 + t) % 1009
                out.append(h % 97)
        return out

    def step(self):
        sched = self.sched
        if self.flight is None:
            batch, dropped = sched.schedule()
            self.returned += dropped
            if not batch:
                return
            self.flight = self._launch(batch)
        cur = self.flight
        tokens = self._tokens(cur)           # known to the device only until resolve
        self.returned += sched.advance(cur)
        batch, dropped = sched.schedule()
        self.returned += dropped
        following = self._launch(batch) if batch else None
        in_next = {s.request.request_id for s in batch}
        self.returned += sched.resolve(cur, tokens, in_next)
        self.flight = following
        self.cache.check()

    def idle(self):
        return self.flight is None and self.sched.is_finished()


def test_eos_on_a_request_preempted_while_its_token_was_under_way_ends_it_once():
    # 3 requests of 8 tokens, pages of 4, 6 pages: the youngest is preempted when the others
    # need their third page, while its first token is still being chosen; that token is its EOS
    reqs = [_req(i, 8, max_tokens=12, ignore_eos=(i != 2)) for i in range(3)]
    eos = _PipelinedHost._tokens([type("S", (), dict(request=reqs[2], start=0, num_tokens=8,
                                                     sample=True))()])[0]
    sched, cache = _sched(pages=6, page=4, seqs=4, budget=64, max_len=24, eos=(eos,))
    for r in reqs:
        sched.add(r)
    host = _PipelinedHost(sched, cache)
    seen_waiting_finished = False
    for _ in range(100):
        if host.idle():
            break
        host.step()
        seen_waiting_finished |= any(r.state is RequestState.FINISHED for r in sched.waiting)
    assert host.idle()
    v = reqs[2]
    assert v.finish_reason == "eos" and v.output == [eos]
    assert host.returned.count(v) == 1 and not seen_waiting_finished
    assert v.num_preemptions >= 1                     # the order the test is about did happen
    assert cache.free_pages() == [6] and cache.slots.num_free == 4


def test_a_request_that_cannot_fit_even_alone_ends_with_out_of_pages():
    sched, cache = _sched(pages=3, page=4, budget=32, max_len=64)
    a = _req(0, 10, max_tokens=30)
    sched.add(a)
    steps = 0
    while not sched.is_finished():
        _run_step(sched, cache)
        steps += 1
        assert steps < 100
    assert a.finish_reason == "out_of_pages" and a.state is RequestState.FINISHED
    assert a.num_tokens == 12 + 1                     # 12 tokens cached, the 13th has no page
    assert cache.free_pages() == [3]


def test_slots_bound_the_live_requests_and_admission_is_in_order():
    sched, cache = _sched(pages=64, seqs=2, budget=64, max_len=64)
    reqs = [_req(i, 5, max_tokens=3) for i in range(5)]
    for r in reqs:
        sched.add(r)
    order = []
    while not sched.is_finished():
        batch, _ = _run_step(sched, cache)
        assert len(sched.running) <= 2
        for s in batch:
            if s.start == 0 and s.request.request_id not in order:
                order.append(s.request.request_id)
    assert order == [0, 1, 2, 3, 4]


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_finish_with_the_results_of_each_request_alone(seed):
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    pages = rng.choice([10, 14, 40])
    windows = rng.choice([(0,), (0, 12)])
    budget = rng.choice([5, 16, 64])
    max_len = pages * page
    reqs = [_req(i, rng.randint(1, min(30, (pages - 1) * page)), max_tokens=rng.randint(1, 12))
            for i in range(rng.randint(3, 9))]
    alone = []
    for r in reqs:
        s2, c2 = _sched(pages=pages, page=page, seqs=3, budget=budget, max_len=max_len,
                        windows=windows)
        clone = Request(r.request_id, list(r.prompt), r.params)
        s2.add(clone)
        while not s2.is_finished():
            _run_step(s2, c2)
        alone.append((list(clone.output), clone.finish_reason))
    sched, cache = _sched(pages=pages, page=page, seqs=3, budget=budget, max_len=max_len,
                          windows=windows)
    pending = list(reqs)
    steps = 0
    while pending or not sched.is_finished():
        while pending and rng.random() < 0.5:
            sched.add(pending.pop(0))
        batch, _ = _run_step(sched, cache)
        assert sum(s.num_tokens for s in batch) <= budget and len(sched.running) <= 3
        steps += 1
        assert steps < 2000, "the scheduler does not make progress"
    for r, (out, why) in zip(reqs, alone):
        if why != "out_of_pages" and r.finish_reason != "out_of_pages":
            assert r.output == out and r.finish_reason == why
    assert cache.free_pages() == [pages] * len(windows) and cache.slots.num_free == 3


def test_sampling_numbers_depend_on_seed_and_index_only():
    assert uniform(3, 5) == uniform(3, 5)
    xs = [uniform(1, i) for i in range(2000)]
    assert all(0.0 <= x < 1.0 for x in xs) and len(set(xs)) > 1990
    assert abs(sum(xs) / len(xs) - 0.5) < 0.03
    assert uniform(1, 7) != uniform(2, 7)


@pytest.mark.parametrize("seed", range(12))
def test_native_decisions_are_the_python_decisions(seed):
    """The same arrivals on a scheduler over the C++ manager (decisions taken in C++) and on one
    over the Python manager (decisions taken in Python), pools so small that requests are
    preempted and given up: the same batch at every step, the same preemptions, the same ends."""
    rng = random.Random(500 + seed)
    page = rng.choice([1, 4, 8])
    pages = rng.choice([5, 9, 14])
    windows = rng.choice([(0,), (0, 6), (0, 5, 13)])
    budget = rng.choice([3, 8, 16])
    max_len = pages * page
    plan = [(i, rng.randint(1, min(30, (pages - 1) * page)), rng.randint(1, 12), rng.randint(0, 3))
            for i in range(rng.randint(3, 10))]
    logs = []
    for manager in (PyCacheManager, NativeCacheManager):
        cache = manager(list(windows), pages, page, 3, max_len)
        native = manager is NativeCacheManager
        sched = (Scheduler if native else PythonScheduler)(cache, 3, budget, max_len, ())
        assert hasattr(cache, "decide") == native
        reqs = [_req(i, n, max_tokens=mt) for i, n, mt, _ in plan]
        pending = list(zip(reqs, (gap for *_, gap in plan)))
        log, steps = [], 0
        while pending or not sched.is_finished():
            while pending and pending[0][1] <= 0:
                sched.add(pending.pop(0)[0])
            if pending:
                pending[0] = (pending[0][0], pending[0][1] - 1)
            _, done = _run_step(sched, cache, log)
            log.append(sorted((r.request_id, r.finish_reason) for r in done))
            log.append([r.request_id for r in sched.running] + ["|"] +
                       [r.request_id for r in sched.waiting])
            steps += 1
            assert steps < 3000
        logs.append((log, sched.num_preemptions,
                     [(r.output, r.finish_reason, r.num_preemptions) for r in reqs]))
    assert logs[0] == logs[1]


def test_batch_sizes_of_decode_graphs():
    """Decode steps are replayed from a graph of their own batch size up to 8 requests, of the
    next multiple of 8 up to 64 and of 16 above (the rows in between are padding)."""
    from ginfer_b200.engine.runner import ModelRunner
    sizes = [ModelRunner.graph_batch(b) for b in range(1, 100)]
    assert sizes[:8] == list(range(1, 9))
    assert all(s >= b and s - b < (8 if b <= 64 else 16) for b, s in zip(range(1, 100), sizes))
    assert sorted(set(sizes)) == list(range(1, 9)) + [16, 24, 32, 40, 48, 56, 64, 80, 96, 112]


def test_split_choices_of_the_kernels():
    """How the decode attention splits a request's keys and the small products their reduction:
    powers of two up to 8 (they form a thread-block cluster), more splits for fewer requests, none
    where the grid fills the GPU anyway; 12 splits for a long reduction on few tiles."""
    from ginfer_b200.ops import attention_bf16, gemm_bf16
    assert attention_bf16.decode_splits(8, 12, 2, 576) == 8
    assert attention_bf16.decode_splits(64, 12, 2, 576) == 2
    assert attention_bf16.decode_splits(512, 12, 2, 576) == 1
    assert attention_bf16.decode_splits(1, 12, 2, 40) == 1           # one tile of keys
    assert attention_bf16.decode_splits(48, 12, 2, 576) == 2         # 4 would not fit at once
    assert attention_bf16.decode_splits(24, 12, 2, 576) == 4
    for b in (1, 3, 8, 20, 64, 200):
        for keys in (10, 600, 5000):
            assert attention_bf16.decode_splits(b, 28, 4, keys) in (1, 2, 4, 8)
    assert attention_bf16.tma_serves(128, 16, 8) and attention_bf16.tma_serves(64, 128, 1)
    assert not attention_bf16.tma_serves(48, 16, 8) and not attention_bf16.tma_serves(128, 24, 2)
    assert not attention_bf16.tma_serves(128, 16, 5)
    assert gemm_bf16.split_k_for(8, 2048, 1536) == 8                 # q/k/v: 16 tiles
    assert gemm_bf16.split_k_for(8, 1536, 8960) == 12                # down: 12 tiles, long K
    assert gemm_bf16.split_k_for(8, 17920, 1536) == 2                # gate/up: about a tile an SM
    assert gemm_bf16.split_k_for(8, 151936, 1536) == 1               # the head: tiles for all SMs
    assert gemm_bf16.split_k_for(64, 17920, 1536) == 2               # still two: more bytes under way
    assert gemm_bf16.split_k_for(128, 17920, 1536) == 1
    # the choices follow the device's SM count, which is asked of the device, not written down
    assert gemm_bf16.num_sms() == gemm_bf16.B200_SMS                 # no device here: a B200's
    assert gemm_bf16.split_k_for(8, 17920, 1536, sms=64) == 1        # 140 tiles on 64 SMs: none
    assert gemm_bf16.split_k_for(8, 1536, 8960, sms=64) == 4         # fewer SMs, fewer splits
    assert attention_bf16.decode_splits(64, 12, 2, 576, sms=32) == 1
    # several clusters a request: only where one cluster leaves most of the GPU idle (few requests,
    # many keys), and never so many that a CTA is left with less than 256 keys (1,024 where one
    # cluster a request fills half of the SMs already)
    P = attention_bf16.decode_partition
    assert P(1, 12, 2, 576) == (8, 1)
    assert P(1, 12, 2, 4096) == (8, 2)
    assert P(1, 12, 2, 32768) == (8, 16)
    assert P(8, 12, 2, 4096) == (8, 1)               # 128 CTAs already
    assert P(8, 12, 2, 32768) == (8, 2)
    assert P(64, 12, 2, 32768) == (2, 1)
    assert P(1, 28, 4, 32768) == (8, 9)              # 4 kv heads: 296 // 32
    for b in (1, 2, 5, 8, 33, 64):
        for keys in (1, 70, 600, 5000, 40000):
            splits, parts = P(b, 12, 2, keys)
            assert parts == 1 or (splits == 8 and keys // (splits * parts) >= 256)
            assert 1 <= parts <= attention_bf16.MAX_PARTS


def test_pages_a_cache_group_can_hold_at_once():
    """A windowed group is never given more pages than its requests can keep live (the pages
    that still hold a position inside some request's window, plus one step's new tokens); a
    group that keeps every position can hold every slot filled to the limit."""
    from ginfer_b200.cache.storage import GroupLayout
    full = GroupLayout(((2, 16), (2, 16)), True, 0, (0, 1))
    win = GroupLayout(((2, 16), (2, 16)), True, 48, (2,))
    assert full.pages_for(4, 256, 64, 16) == 4 * 16
    # window 48 on pages of 16: positions len-47 .. len-1 touch at most 4 pages, one more while a
    # step's tokens are reserved before the old pages are given back; 64 new tokens take 4 pages
    assert win.pages_for(4, 256, 64, 16) == 4 * 5 + 4
    assert win.pages_for(4, 32, 64, 16) == 4 * 2                    # never more than a full group
    assert full.bytes_per_page(16, 2) == 2 * 16 * 64 * 2 and win.bytes_per_page(16, 2) == 16 * 64 * 2
    # the bound holds for the cache manager's own rules, whatever the portions
    import random
    rng = random.Random(0)
    for page, window, seqs, budget in ((4, 9, 3, 7), (8, 48, 4, 32), (16, 70, 2, 200), (4, 4, 5, 64)):
        g = GroupLayout(((1, 8),) * 2, True, window, (0,))
        cap = g.pages_for(seqs, 4096, budget, page)
        m = _MANAGER[0]([window], cap, page, seqs, 4096)
        for i in range(seqs):
            m.admit(i)
        for _ in range(300):
            left = budget
            step = []
            for i in rng.sample(range(seqs), seqs):
                n = rng.randint(0, left)
                if n:
                    step.append((i, n))
                    left -= n
            for i, n in step:
                m.reserve(i, n)                                      # never out of pages
            for i, n in step:
                m.commit(i, n)
            m.check()
            for i in range(seqs):
                if m.get(i).num_tokens > 3000:
                    m.release(i)
                    m.admit(i)


def test_the_q_k_v_epilogue_is_only_offered_what_it_takes():
    """The product that rotates q/k and writes the cache in its epilogue hands back every case it
    does not serve (the plain product and the rotation kernel run then): few tokens, other head
    sizes, a partly rotated head, no rotation, 32-bit operands, tables or pages of another type;
    and it refuses tensors that are not on a CUDA device instead of handing their addresses to a
    kernel."""
    import pytest
    import torch

    from ginfer_b200.ops import gemm_prefill
    nh, nkv, hd, M, K = 4, 2, 64, 2048, 128
    N = (nh + 2 * nkv) * hd
    x = torch.zeros(M, K, dtype=torch.bfloat16)
    w = torch.zeros(N, K, dtype=torch.bfloat16)
    table = torch.zeros(16, hd)
    pos = torch.zeros(M, dtype=torch.int32)
    pages = torch.zeros(2, 4, 16, nkv, hd, dtype=torch.bfloat16)

    def offered(**kw):
        a = dict(x=x, weight=w, table=table, rot=hd, positions=pos, slot_mapping=pos, pages=pages,
                 nh=nh, nkv=nkv, hd=hd, min_tokens=gemm_prefill.QKV_MIN_TOKENS)
        a.update(kw)
        return gemm_prefill.qkv_epilogue_serves(**a)
    assert offered()
    assert not offered(x=x[:1000])                                         # fewer than 1,024 tokens
    assert offered(x=x[:1000], min_tokens=1)
    assert not offered(x=x.float()) and not offered(table=table.double())
    assert not offered(rot=hd // 2, table=torch.zeros(16, hd // 2))        # a partly rotated head
    assert not offered(table=None, rot=0)
    assert not offered(slot_mapping=None)                                   # a run that does not write
    assert not offered(pages=pages.float()) and not offered(pages=pages[:, :, :, :1])
    assert not offered(positions=pos.long()) and not offered(slot_mapping=pos[:5])
    assert not offered(hd=32, nh=8, nkv=4, table=torch.zeros(16, 32), rot=32,
                       pages=torch.zeros(2, 4, 16, 4, 32, dtype=torch.bfloat16))
    assert not offered(weight=w[:-hd]) and not offered(weight=w.float())    # rows that are no heads
    with pytest.raises(RuntimeError, match="CUDA device only"):
        gemm_prefill.qkv_rope_write(x, w, None, table, hd, pos, pos, pages, nh, nkv, hd,
                                    min_tokens=1)
    with pytest.raises(RuntimeError, match="CUDA device only"):
        gemm_prefill.gemm(x, w)


def test_the_reference_benchmark_workload_is_scheduled_in_nine_prompt_steps():
    """256 prompts of 512 tokens, 128 tokens generated for each, a budget of 16,384 tokens a step
    and 256 requests at a time (the reference's own throughput run): about 32 prompts a step,
    while the requests admitted earlier decode beside them, then decode steps of all 256; nobody
    is preempted and every page and slot comes back."""
    page = 16
    sched, cache = _sched(pages=256 * (640 // page + 2), page=page, seqs=256, budget=16384,
                          max_len=4096)
    reqs = [Request(i, [(i + j) % 97 for j in range(512)],
                    SamplingParams(max_tokens=128, ignore_eos=True)) for i in range(256)]
    for r in reqs:
        sched.add(r)
    steps, prompt_steps = 0, 0
    while not sched.is_finished():
        batch, dropped = sched.schedule()
        assert not dropped and batch
        assert sum(s.num_tokens for s in batch) <= 16384 and len(batch) <= 256
        for s in batch:
            cache.reserve(s.request.request_id, s.num_tokens)
        for s in batch:
            cache.commit(s.request.request_id, s.num_tokens)
        prompt_steps += any(s.num_tokens > 1 for s in batch)
        sched.postprocess(batch, [5] * sum(1 for s in batch if s.sample))
        steps += 1
        assert steps < 400
    cache.check()
    # 131,072 prompt tokens are eight budgets, but the requests that decode already take their
    # token of each step's budget first: the last prompts spill into a ninth step
    assert prompt_steps == 9
    assert all(len(r.output) == 128 and r.finish_reason == "max_tokens" for r in reqs)
    assert sched.num_preemptions == 0
    assert cache.free_pages() == [256 * (640 // page + 2)] and cache.slots.num_free == 256


def test_the_bench_scenarios_fit_the_engines_they_ask_for():
    """Every prompt of a serving workload of ``bench.py``, with the tokens it generates, fits the
    engine's longest sequence and the model's position table, at every shape (the runner takes
    the smaller of the two as its limit and refuses longer requests)."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    for name in bench.SCENARIOS:
        if name == "longctx":
            continue                                     # (one prompt, sized from its arguments)
        for shape in bench.SHAPES:
            cfg, full_layers, prompts, params, kwargs = bench.scenario_plan(name, shape, 2)
            limit = min(kwargs["max_seq_len"], cfg["max_position_embeddings"])
            longest = max(len(p) + q.max_tokens for p, q in zip(prompts, params))
            assert longest <= limit, (name, shape, longest, limit)
            assert len(prompts) == len(params) and cfg["num_hidden_layers"] == 2
            assert full_layers == bench.SHAPES[shape]["num_hidden_layers"]
            # pages for every request at its full length, so that nobody is preempted
            pages = sum(-(-(len(p) + q.max_tokens) // bench.PAGE) for p, q in zip(prompts, params))
            assert pages <= kwargs["num_kvcache_blocks"], (name, shape, pages)
