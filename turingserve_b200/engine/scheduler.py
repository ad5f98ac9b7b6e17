"""Scheduler: continuous batching with chunked prefill under a token budget, decodes first,
recompute preemption when pages run out.

The three passes and every decision in them follow turingserve/scheduler/scheduler.py:65-130:

1. every running request with exactly one uncomputed token decodes, oldest first; if its page does
   not fit, the NEWEST running request that is not yet in the plan is preempted (or the request
   itself when there is no other), until it fits (:72-94);
2. running requests in the middle of a prompt get min(uncomputed, budget) tokens; if the pages do
   not fit the pass stops; nothing is preempted for a prompt portion (:96-106), except when no
   request at all could run: then the newest running request is preempted, and a request that is
   stuck alone (its prompt cannot fit the pool) is handed back as failed;
3. waiting requests are admitted first-come first-served while budget, request slots and pages
   (leaving a watermark free) allow, and only if this step preempted nothing (:108-124).

Preemption is by recompute (:43-55): the victim's pages and state slot go back, it returns to the
FRONT of the waiting queue, and its generated tokens are prefilled again like prompt tokens.
A request that cannot fit even in an empty pool is reported by ``unschedulable()`` so the engine
can finish it with an error (turingserve/engine/engine.py:199-208).
"""

from __future__ import annotations

from collections import deque

from turingserve_b200.cache.manager import CacheManager
from turingserve_b200.engine.request import BatchPlan, Request, Scheduled, Status


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_batched_tokens: int, max_num_seqs: int,
                 watermark: float = 0.01) -> None:
        self.cache = cache
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_num_seqs = min(max_num_seqs, cache.max_requests)
        usable = min((g.allocator.num_usable for g in cache.groups), default=0)
        self.watermark_pages = max(1, int(watermark * (usable + 1))) if cache.groups else 0
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.num_preemptions = 0

    # -- queues -----------------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        req.status = Status.WAITING
        self.waiting.append(req)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def finish(self, req: Request) -> None:
        """Remove a finished or aborted request and give back what it holds."""
        if req in self.running:
            self.running.remove(req)
        else:
            try:
                self.waiting.remove(req)
            except ValueError:
                pass
        if req.cache is not None:
            self.cache.release(req.cache)
            req.cache = None

    def _preempt(self, req: Request) -> None:
        self.cache.release(req.cache)
        req.cache = None
        req.status = Status.WAITING
        req.num_preemptions += 1
        self.running.remove(req)
        self.waiting.appendleft(req)
        self.num_preemptions += 1

    def preempt_all(self) -> list[Request]:
        victims = list(self.running)
        for r in reversed(victims):
            self._preempt(r)
        return victims

    def unschedulable(self) -> Request | None:
        """The head of the waiting queue, if nothing runs and it can never be admitted."""
        if self.running or not self.waiting:
            return None
        return self.waiting[0]

    # -- one step's plan -------------------------------------------------------------------------
    def schedule(self) -> BatchPlan:
        budget = self.max_num_batched_tokens
        plan: list[Scheduled] = []
        in_plan: set[int] = set()
        preempted: list[Request] = []
        preempted_ids: set[int] = set()
        cache = self.cache

        for req in [r for r in self.running if r.num_uncomputed == 1]:
            if id(req) in preempted_ids or budget <= 0:
                continue
            while not cache.can_grow(req.cache, 1):
                victim = None
                for cand in reversed(self.running):
                    if cand is not req and id(cand) not in in_plan:
                        victim = cand
                        break
                if victim is None:
                    victim = req
                self._preempt(victim)
                preempted.append(victim)
                preempted_ids.add(id(victim))
                if victim is req:
                    break
            if id(req) in preempted_ids:
                continue
            cache.grow(req.cache, 1)
            plan.append(Scheduled(req, 1, True))
            in_plan.add(id(req))
            budget -= 1

        failed: list[Request] = []
        while True:
            for req in [r for r in self.running if r.num_uncomputed > 1 and id(r) not in preempted_ids]:
                if budget == 0:
                    break
                n = min(req.num_uncomputed, budget)
                if not cache.can_grow(req.cache, n):
                    break
                cache.grow(req.cache, n)
                plan.append(Scheduled(req, n, n == req.num_uncomputed))
                in_plan.add(id(req))
                budget -= n
            if plan or not self.running:
                break
            # Nothing can run although requests hold pages: every one of them is a prompt portion
            # that does not fit.  The reference would wait forever here; this engine gives the
            # newest one's pages to the others, and fails a request that is stuck all alone.
            victim = self.running[-1]
            if len(self.running) == 1:
                self.running.remove(victim)
                cache.release(victim.cache)
                victim.cache = None
                failed.append(victim)
                break
            self._preempt(victim)
            preempted.append(victim)
            preempted_ids.add(id(victim))

        while (self.waiting and budget > 0 and not preempted
               and len(self.running) < self.max_num_seqs and cache.has_free_slot()):
            req = self.waiting[0]
            n = min(req.num_uncomputed, budget)
            if not cache.can_grow(None, n, keep_free=self.watermark_pages):
                break
            self.waiting.popleft()
            req.status = Status.RUNNING
            req.cache = cache.admit(req.request_id)
            self.running.append(req)
            cache.grow(req.cache, n)
            plan.append(Scheduled(req, n, n == req.num_uncomputed))
            budget -= n

        def is_decode(p: Scheduled) -> bool:
            return p.num_tokens == 1 and p.request.num_uncomputed == 1

        decodes = [p for p in plan if is_decode(p)]
        prefills = [p for p in plan if not is_decode(p)]
        items = decodes + prefills
        return BatchPlan(items=items, num_decode=len(decodes),
                         num_tokens=sum(p.num_tokens for p in items), preempted=preempted,
                         failed=failed)
