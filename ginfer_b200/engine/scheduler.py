"""Continuous batching with prompts fed in portions under a token budget.

Reference: ``ginfer/engine/scheduler.cc:20-99``.  There a step is either all prompts (each whole)
or all decode tokens; a prompt longer than the budget is never scheduled; when a decoding request
cannot get a page the most recently admitted running request is preempted (its pages released,
itself queued again and later computed from the start, ``scheduler.cc:47-56,73-77``); a request
finishes on an EOS id (unless ``ignore_eos``) or at ``max_tokens`` (``scheduler.cc:83-98``).

Here every step is one mixed batch, built in this order:

1. every running request that is decoding gets its one token;
2. running requests still in their prompt get a portion of it;
3. waiting requests are admitted, oldest first, while a slot, budget and pages for a first
   portion are there (a request that does not fit stops admission: no overtaking).

The budget is ``max_num_batched_tokens`` tokens a step; a portion is whatever of the prompt is
left, cut to the budget and to the pages that are free.

When pages run out: a decoding request that needs a page takes it from the most recently admitted
other running request, which is preempted: its pages go back, it keeps its slot and its sampling
state, it is put at the *front* of the waiting queue and is later computed again from its first
token (prompt and the output so far).  A request that is alone and still cannot get a page is
finished with reason ``out_of_pages``; a prompt that could never fit the pool or ``max_seq_len``
is refused when it is added.  Nothing spins.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass

from ..cache import NativeCacheManager as CacheManager
from .request import Request, RequestState


@dataclass
class Scheduled:
    request: Request
    start: int            # position of the first token of the portion
    num_tokens: int
    sample: bool          # the portion ends at the request's last token: a token is sampled
    dropped: bool = False  # the request had ended already when this step was advanced


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int,
                 max_seq_len: int, eos_token_ids=()):
        self.cache = cache
        self.max_num_seqs = int(max_num_seqs)
        self.max_num_batched_tokens = int(max_num_batched_tokens)
        self.max_seq_len = int(max_seq_len)
        self.eos = frozenset(int(e) for e in eos_token_ids)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []          # in order of admission
        self.num_preemptions = 0

    # ------------------------------------------------------------------ queue
    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, req: Request) -> None:
        n = len(req.prompt)
        if n == 0:
            raise ValueError("a prompt needs at least one token")
        if n + 1 > self.max_seq_len:
            raise ValueError(f"prompt of {n} tokens leaves no room for output within "
                             f"max_seq_len {self.max_seq_len}")
        need = -(-n // self.cache.page_size)
        for g, pool in enumerate(self.cache.pools):
            if need > pool.num_pages and self.cache.windows[g] == 0:
                raise ValueError(f"prompt of {n} tokens needs {need} pages; the pool of group "
                                 f"{g} has {pool.num_pages}")
        req.state = RequestState.WAITING
        self.waiting.append(req)

    # ------------------------------------------------------------------ one step
    def _finish(self, req: Request, reason: str) -> None:
        req.state = RequestState.FINISHED
        req.finish_reason = reason
        req.finish_time = time.perf_counter()
        if req in self.running:
            self.running.remove(req)
        if req in self.waiting:
            # preempted while its last token was still under way, and that token ended it: a
            # request left here would be admitted and computed again
            self.waiting.remove(req)
        if self.cache.has(req.request_id):
            self.cache.release(req.request_id)

    def schedule(self) -> tuple[list[Scheduled], list[Request]]:
        """Returns the step's batch and the requests finished without a step (out of pages).
        The decision itself (the three rules above, preemption included) is taken in C++ in one
        call: ``gf_sched_decide`` in ``csrc/cache_core.cu``."""
        reqs = list(self.running) + list(self.waiting)
        nr = len(self.running)
        acts, running, waiting, preempts, dropped = self.cache.decide(
            self.max_num_batched_tokens, self.max_num_seqs,
            [(r.request_id, r.num_tokens, r.num_computed) for r in reqs[:nr]],
            [(r.request_id, r.num_tokens, r.num_computed) for r in reqs[nr:]])
        out: list[Request] = []
        for e, req in enumerate(reqs):
            if preempts[e]:
                req.num_computed = 0
                req.num_preemptions += preempts[e]
                self.num_preemptions += preempts[e]
            if dropped[e]:
                req.state = RequestState.FINISHED
                req.finish_reason = "out_of_pages"
                req.finish_time = time.perf_counter()
                out.append(req)
        self.running = [reqs[e] for e in running]
        self.waiting = deque(reqs[e] for e in waiting)
        for r in self.running:
            r.state = RequestState.RUNNING
        for r in self.waiting:
            r.state = RequestState.WAITING
        return [Scheduled(reqs[e], start, n, bool(sample)) for e, start, n, sample in acts], out

    def postprocess(self, batch: list[Scheduled], sampled: list[int]) -> list[Request]:
        """``sampled``: one token for every entry of ``batch`` with ``sample`` set, in order.
        Appends tokens, finishes requests, returns the finished ones."""
        finished = self.advance(batch)
        finished += self.resolve(batch, sampled)
        return finished

    # The two halves of post-processing, for a host that prepares the next step while the
    # device still runs this one.  ``advance`` needs no token values: it moves the requests
    # forward, appends a placeholder for each token being sampled, and finishes what is finished
    # by count.  ``resolve`` fills the placeholders in once the tokens are known and applies the
    # EOS rule; a request that is already part of a step in preparation (``in_next``) is only
    # marked and finishes when that step is advanced (its extra token is dropped).
    PENDING = -1

    def advance(self, batch: list[Scheduled]) -> list[Request]:
        finished = []
        for s in batch:
            req = s.request
            if req.finish_pending is not None:        # hit EOS one step ago: this step is dropped
                reason, req.finish_pending = req.finish_pending, None
                s.dropped = True
                self._finish(req, reason)
                finished.append(req)
                continue
            req.num_computed = s.start + s.num_tokens
            if not s.sample:
                continue
            req.output.append(self.PENDING)
            if len(req.output) >= req.params.max_tokens:
                self._finish(req, "max_tokens")
            elif req.num_tokens >= self.max_seq_len:
                self._finish(req, "max_seq_len")
            if req.state is RequestState.FINISHED:
                finished.append(req)
        return finished

    def resolve(self, batch: list[Scheduled], sampled: list[int], in_next=()) -> list[Request]:
        finished = []
        it = iter(sampled)
        now = time.perf_counter()
        for s in batch:
            if not s.sample:
                continue
            tok = int(next(it))
            if s.dropped:
                continue
            req = s.request
            idx = s.start + s.num_tokens - len(req.prompt)       # the output index of this token
            req.output[idx] = tok
            if req.first_token_time is None:
                req.first_token_time = now
            if not req.params.ignore_eos and tok in self.eos:
                if req.state is RequestState.FINISHED:
                    req.finish_reason = "eos"                     # by count as well: EOS names it
                elif req.request_id in in_next:
                    req.finish_pending = "eos"
                else:
                    self._finish(req, "eos")
                    finished.append(req)
        return finished
