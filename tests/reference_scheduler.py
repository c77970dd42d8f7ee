"""The scheduler's decision in plain Python: the oracle that the tests compare the C++ decision
(``gf_sched_decide`` in ``ginfer_b200/csrc/cache_core.cu``, the one the engine runs) with, step
by step.  Not part of the product.  The rules are those in the header of
``ginfer_b200/engine/scheduler.py``."""
from __future__ import annotations

from ginfer_b200.engine.request import Request, RequestState
from ginfer_b200.engine.scheduler import Scheduled, Scheduler


class PythonScheduler(Scheduler):
    """:class:`Scheduler` with the decision of a step taken here instead of in native code; works
    over either cache manager."""

    def schedule(self) -> tuple[list[Scheduled], list[Request]]:
        return self._schedule_python()

    def _fit(self, req: Request, want: int, promised: list[int]) -> int:
        """Largest portion <= ``want`` whose pages are free (beyond ``promised``)."""
        if want <= 0:
            return 0
        if self.cache.can_reserve(req.request_id, want, promised):
            return want
        P = self.cache.page_size
        have = req.num_computed
        free = min(f - p for f, p in zip(self.cache.free_pages(), promised))
        if free < 0:
            return 0
        # tokens until the pages held so far are full, plus what ``free`` more pages hold
        rc = self.cache.requests.get(req.request_id)
        held_end = (min(rc.next_page) if rc else 0) * P
        room = max(0, held_end - have) + free * P
        n = min(want, room)
        while n > 0 and not self.cache.can_reserve(req.request_id, n, promised):
            n -= 1
        return n

    def _need_fits(self, need: list[int], promised: list[int]) -> bool:
        """Whether ``need`` pages per group are free beyond what is ``promised`` to others."""
        if not any(need):
            return True
        return all(k <= f - p for k, f, p in zip(need, self.cache.free_pages(), promised))

    def _promise(self, req: Request, n: int, promised: list[int]) -> None:
        for g, k in enumerate(self.cache.pages_needed(req.request_id, n)):
            promised[g] += k

    def _preempt(self, victim: Request) -> None:
        self.cache.release(victim.request_id, keep_slot=True)
        victim.num_computed = 0
        victim.state = RequestState.WAITING
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(victim)
        self.waiting.appendleft(victim)

    def _schedule_python(self) -> tuple[list[Scheduled], list[Request]]:
        budget = self.max_num_batched_tokens
        promised = [0] * self.cache.num_groups
        batch: list[Scheduled] = []
        dropped: list[Request] = []

        # 1. decoding requests, oldest first; a page may cost the youngest its place
        for req in list(self.running):
            if req.state is not RequestState.RUNNING or req.num_tokens - req.num_computed != 1:
                continue
            if budget <= 0:
                break
            need = self.cache.pages_needed(req.request_id, 1)    # preempting others leaves it as is
            while not self._need_fits(need, promised):
                victims = [r for r in self.running if r is not req
                           and all(s.request is not r for s in batch)]
                if victims:
                    self._preempt(victims[-1])
                elif len(self.running) > 1 or batch:
                    break                      # others already hold this step's pages: wait
                else:
                    self._finish(req, "out_of_pages")
                    dropped.append(req)
                    break
            if req.state is not RequestState.RUNNING or not self._need_fits(need, promised):
                continue
            for g, k in enumerate(need):
                promised[g] += k
            batch.append(Scheduled(req, req.num_computed, 1, True))
            budget -= 1

        # 2. running requests still feeding their prompt
        for req in list(self.running):
            left = req.num_tokens - req.num_computed
            if req.state is not RequestState.RUNNING or left <= 1 or budget <= 0:
                continue
            n = self._fit(req, min(left, budget), promised)
            if n <= 0:
                continue
            self._promise(req, n, promised)
            batch.append(Scheduled(req, req.num_computed, n, n == left))
            budget -= n

        # 3. admission, oldest first, no overtaking
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            if not self.cache.has(req.request_id) and self.cache.slots.num_free == 0:
                break
            left = req.num_tokens
            n = self._fit(req, min(left, budget), promised)
            if n <= 0:
                break
            self.waiting.popleft()
            if not self.cache.has(req.request_id):
                self.cache.admit(req.request_id)
            req.state = RequestState.RUNNING
            self.running.append(req)
            self._promise(req, n, promised)
            batch.append(Scheduled(req, 0, n, n == left))
            budget -= n

        # nothing could move although requests are live: free the youngest's pages, or give up on
        # a request that is alone
        if not batch and not dropped and (self.running or self.waiting):
            if len(self.running) > 1:
                self._preempt(self.running[-1])
                return self._schedule_python()
            if self.running:
                req = self.running[0]
                self._finish(req, "out_of_pages")
                dropped.append(req)
            elif self.waiting:
                req = self.waiting.popleft()
                self._finish(req, "out_of_pages")
                dropped.append(req)
        return batch, dropped

