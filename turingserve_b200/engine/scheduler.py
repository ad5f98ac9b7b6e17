"""Scheduler: which requests run in the next step, and with how many tokens each.

Behaviour (continuous batching with prompts cut into portions under a token budget, decodes
before prompts, recompute preemption) is the reference's, turingserve/scheduler/scheduler.py:65-130;
the structure is this engine's: a step is drafted by three methods, one per kind of work, that share
a ``_Draft`` (budget left, portions taken, requests evicted).

1. ``_take_decodes``: every running request with one token to run gets it, oldest first.  When its
   next page does not fit, room is made by evicting the NEWEST running request that has no portion
   in the draft yet; a request that would have to evict itself is evicted and skipped (:72-94).
2. ``_take_running_prompts``: running requests in the middle of a prompt get as much as the budget
   allows, in order, until one does not fit; nothing is evicted for a prompt portion (:96-106).
   Beyond the reference: if after this nothing at all is drafted although requests hold pages (every
   one of them a prompt portion that cannot grow), the newest gives up its pages and the pass runs
   again; a request that is stuck alone can never fit and is handed back in ``StepPlan.failed``.
3. ``_admit``: waiting requests are admitted first come first served while budget, request slots and
   pages (less a watermark) last; not in a step that evicted someone (:108-124).

Eviction is by recompute (:43-55): pages and state slot go back, the request returns to the FRONT
of the queue and runs its prompt and its own output again as one long prompt.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from turingserve_b200.cache.manager import CacheManager
from turingserve_b200.engine.request import Request, Status


@dataclass
class Portion:
    """A request's share of a step."""

    request: Request
    num_tokens: int
    samples: bool              # it reaches the request's last token, so the step draws its next one


@dataclass
class StepPlan:
    items: list[Portion] = field(default_factory=list)           # single decoded tokens first
    num_decode: int = 0
    num_tokens: int = 0
    preempted: list[Request] = field(default_factory=list)
    failed: list[Request] = field(default_factory=list)          # can never fit: to be finished with "error"


class _Draft:
    """A step while it is being put together."""

    def __init__(self, budget: int) -> None:
        self.budget = budget
        self.decodes: list[Portion] = []
        self.prompts: list[Portion] = []
        self.taken: set[int] = set()               # id() of requests that have a portion
        self.evicted: list[Request] = []
        self.failed: list[Request] = []

    def take(self, req: Request, n: int) -> None:
        portion = Portion(req, n, samples=(n == req.num_uncomputed))
        (self.decodes if req.decoding and n == 1 else self.prompts).append(portion)
        self.taken.add(id(req))
        self.budget -= n

    def was_evicted(self, req: Request) -> bool:
        return any(v is req for v in self.evicted)

    def empty(self) -> bool:
        return not self.decodes and not self.prompts

    def plan(self) -> StepPlan:
        items = self.decodes + self.prompts
        return StepPlan(items, len(self.decodes), sum(p.num_tokens for p in items), self.evicted, self.failed)


class Scheduler:
    SMALLEST_CAPTURED_PORTION = 16      # shorter prompt portions than this get no captured step shape

    def __init__(self, cache: CacheManager, max_num_batched_tokens: int, max_num_seqs: int,
                 watermark: float = 0.01, padded_decodes=None) -> None:
        """``padded_decodes``: n -> the number of rows the runner fills n decoding requests up to (None: it
        does not); those rows count against the token budget, so that a prompt portion beside them has one
        of a few lengths and the step one of a few captured shapes."""
        self.cache = cache
        self.padded_decodes = padded_decodes
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_num_seqs = min(max_num_seqs, cache.max_requests)
        smallest_pool = min((g.allocator.num_usable for g in cache.groups), default=0)
        self.watermark_pages = max(1, int(watermark * (smallest_pool + 1))) if cache.groups else 0
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []           # in order of admission: the newest is last
        self.num_preemptions = 0

    # -- the queues ---------------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        req.status = Status.WAITING
        self.waiting.append(req)

    def has_unfinished(self) -> bool:
        return len(self.waiting) + len(self.running) > 0

    def finish(self, req: Request) -> None:
        """A request has ended (finished or aborted): out of whichever queue holds it, pages back."""
        for queue in (self.running, self.waiting):
            if req in queue:
                queue.remove(req)
                break
        self._give_back(req)

    def unschedulable(self) -> Request | None:
        """With nothing running and a step that came out empty, the head of the queue is a request
        that does not fit even an empty pool."""
        if self.running or not self.waiting:
            return None
        return self.waiting[0]

    def preempt_all(self) -> list[Request]:
        """Evict everything that runs, newest first, so the queue keeps the order of admission."""
        victims = self.running[:]
        for req in victims[::-1]:
            self._evict(req)
        return victims

    def _give_back(self, req: Request) -> None:
        if req.cache is not None:
            self.cache.release(req.cache)
            req.cache = None

    def _evict(self, req: Request, draft: _Draft | None = None) -> None:
        self.running.remove(req)
        self._give_back(req)
        req.status = Status.WAITING
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)
        if draft is not None:
            draft.evicted.append(req)

    # -- one step ------------------------------------------------------------------------------------
    def schedule(self) -> StepPlan:
        draft = _Draft(self.max_num_batched_tokens)
        self._take_decodes(draft)
        if self.padded_decodes is not None and draft.decodes:
            rows = self.padded_decodes(len(draft.decodes))
            # (not where the padding would leave a prompt next to nothing: that step is launched kernel by
            # kernel, with all of the budget)
            if rows is not None and draft.budget - (rows - len(draft.decodes)) >= self.SMALLEST_CAPTURED_PORTION:
                draft.budget -= rows - len(draft.decodes)
        self._take_running_prompts(draft)
        if not draft.evicted:
            self._admit(draft)
        return draft.plan()

    def _newest_without_portion(self, draft: _Draft, other_than: Request) -> Request | None:
        for req in self.running[::-1]:
            if req is not other_than and id(req) not in draft.taken:
                return req
        return None

    def _make_room_for_decode(self, req: Request, draft: _Draft) -> bool:
        """Evict until ``req``'s next token has a page; False when ``req`` itself had to go."""
        while not self.cache.can_grow(req.cache, 1):
            victim = self._newest_without_portion(draft, other_than=req) or req
            self._evict(victim, draft)
            if victim is req:
                return False
        return True

    def _take_decodes(self, draft: _Draft) -> None:
        for req in [r for r in self.running if r.decoding]:
            if draft.budget < 1:
                return
            if draft.was_evicted(req):
                continue
            if self._make_room_for_decode(req, draft):
                self.cache.grow(req.cache, 1)
                draft.take(req, 1)

    def _take_running_prompts(self, draft: _Draft) -> None:
        while True:
            for req in [r for r in self.running if not r.decoding]:
                n = min(req.num_uncomputed, draft.budget)
                if n < 1 or not self.cache.can_grow(req.cache, n):
                    break
                self.cache.grow(req.cache, n)
                draft.take(req, n)
            if not draft.empty() or not self.running:
                return
            # Requests hold pages and none of them can move: each is a prompt portion that does not
            # fit.  The newest makes room for the others; alone, it can never fit.
            newest = self.running[-1]
            if len(self.running) == 1:
                self.running.remove(newest)
                self._give_back(newest)
                draft.failed.append(newest)
                return
            self._evict(newest, draft)

    def _admit(self, draft: _Draft) -> None:
        while self.waiting and draft.budget > 0:
            if len(self.running) >= self.max_num_seqs or not self.cache.has_free_slot():
                return
            req = self.waiting[0]
            n = min(req.num_uncomputed, draft.budget)
            if not self.cache.can_grow(None, n, keep_free=self.watermark_pages):
                return
            self.waiting.popleft()
            req.cache = self.cache.admit(req.request_id)
            req.status = Status.RUNNING
            self.running.append(req)
            self.cache.grow(req.cache, n)
            draft.take(req, n)
