"""Cache manager: paged keys/values with one block table per (request, group), and fixed-size
per-request state slots.

Runs of the schedule whose mixers want the same thing from the cache (same kv heads, head size
and window) form a GROUP.  A group has its own pool ``[runs, 2, pages, kv_heads, page, head_dim]``
(the reference's single ``[L, 2, NB, KVH, 16, D]`` tensor, turingserve/engine/builder.py:76-80,
is the one-group case), its own allocator and, per request, its own block table.  Pages go back
to the group's free list when a request is released, and, in a windowed group, as soon as the
window has passed them; freed pages are re-issued first-in first-out.

Slot arithmetic as turingserve/kv/kv_manager.py:17-40:
slot(pos) = table[pos // page] * page + pos % page; pages needed = ceil(tokens / page) - held.

State slots: every live request owns one slot index in [0, max_requests); each run whose mixer
declares a ``StateNeed`` has a tensor ``[max_requests + 1, *shape]`` indexed by it.  A slot is zeroed
when a request is admitted (so recompute after preemption starts clean).  The extra last slot
(``null_slot``) is never handed out: rows that only pad a batch to a captured size point at it, as
their block tables point at the null page.  The reference has no per-request state; the slot is
assigned for every request even when no mixer uses it.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from turingserve_b200.cache.allocator import NoFreePages, PageAllocator
from turingserve_b200.parts.base import CacheNeed, StateNeed


@dataclass(frozen=True)
class RunNeeds:
    """What run ``index`` of the schedule needs: its mixer's cache and state declarations, and
    whose cache it reads when it has none of its own."""

    cache: CacheNeed | None
    state: StateNeed | None
    cache_from: int | None = None


@dataclass
class CacheView:
    """What a mixer sees of the cache for one run."""

    group: int
    k: torch.Tensor | None          # [pages, kv_heads, page, head_dim]
    v: torch.Tensor | None
    page_size: int
    writable: bool                  # False when this run reads another run's cache


@dataclass
class RequestCache:
    """Cache bookkeeping of one live request."""

    request_id: str
    slot: int
    tables: list[list[int]]                       # per group: logical page -> physical page (0 = none)
    num_tokens: int = 0                           # tokens whose keys/values are in the cache
    first_live_page: list[int] = field(default_factory=list)   # per group: pages before it were given back


class CacheGroup:
    def __init__(self, need: CacheNeed, runs: list[int], num_pages: int) -> None:
        self.need = need
        self.runs = runs
        self.allocator = PageAllocator(num_pages)
        self.pool: torch.Tensor | None = None


class CacheManager:
    def __init__(self, needs: list[RunNeeds], page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype = torch.float32, device=None) -> None:
        """``device`` None keeps the bookkeeping only (no tensors): enough for scheduling tests."""
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.dtype, self.device = dtype, device
        self.groups: list[CacheGroup] = []
        self._run_group: list[int | None] = [None] * len(needs)
        self._run_index_in_group: list[int | None] = [None] * len(needs)
        self._needs = needs
        keys: dict[tuple, int] = {}
        for r, n in enumerate(needs):
            if n.cache is None or n.cache_from is not None:
                continue
            key = (n.cache.num_kv_heads, n.cache.head_dim, n.cache.window)
            if key not in keys:
                keys[key] = len(self.groups)
                self.groups.append(CacheGroup(n.cache, [], num_pages))
            g = keys[key]
            self._run_group[r] = g
            self._run_index_in_group[r] = len(self.groups[g].runs)
            self.groups[g].runs.append(r)
        for r, n in enumerate(needs):
            if n.cache_from is not None:
                src = n.cache_from
                if self._run_group[src] is None:
                    raise ValueError(f"run {r} reads the cache of run {src}, which has none")
                a, b = needs[src].cache, n.cache
                if b is not None and (a.num_kv_heads, a.head_dim) != (b.num_kv_heads, b.head_dim):
                    raise ValueError(f"run {r} cannot read run {src}'s cache: different kv shape")
        self.states: list[torch.Tensor | None] = [None] * len(needs)
        if device is not None:
            for grp in self.groups:
                grp.pool = torch.zeros((len(grp.runs), 2, num_pages, grp.need.num_kv_heads, page_size,
                                        grp.need.head_dim), dtype=dtype, device=device)
            for r, n in enumerate(needs):
                if n.state is not None:
                    self.states[r] = torch.zeros((max_requests + 1, *n.state.shape), dtype=n.state.dtype,
                                                 device=device)
        self.null_slot = max_requests
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.live: dict[str, RequestCache] = {}

    # -- sizing -----------------------------------------------------------------------------------
    @staticmethod
    def bytes_per_page(needs: list[RunNeeds], page_size: int, dtype: torch.dtype) -> int:
        """Bytes one page index costs across all groups (each group has ``num_pages`` pages)."""
        elem = torch.empty((), dtype=dtype).element_size()
        return sum(2 * n.cache.num_kv_heads * n.cache.head_dim * page_size * elem
                   for n in needs if n.cache is not None and n.cache_from is None)

    # -- views --------------------------------------------------------------------------------------
    def view(self, run: int) -> CacheView | None:
        n = self._needs[run]
        src = run if n.cache_from is None else n.cache_from
        g = self._run_group[src]
        if g is None:
            return None
        grp = self.groups[g]
        i = self._run_index_in_group[src]
        k = v = None
        if grp.pool is not None:
            k, v = grp.pool[i, 0], grp.pool[i, 1]
        return CacheView(g, k, v, self.page_size, writable=n.cache_from is None)

    def views(self) -> list[CacheView | None]:
        return [self.view(r) for r in range(len(self._needs))]

    # -- requests ---------------------------------------------------------------------------------
    def admit(self, request_id: str) -> RequestCache:
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise NoFreePages("no free state slot")
        slot = self._free_slots.pop()
        for st in self.states:
            if st is not None:
                st[slot].zero_()
        rc = RequestCache(request_id, slot, [[] for _ in self.groups], 0, [0] * len(self.groups))
        self.live[request_id] = rc
        return rc

    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def pages_needed(self, rc: RequestCache, num_new_tokens: int) -> list[int]:
        total = -(-(rc.num_tokens + num_new_tokens) // self.page_size)
        return [max(0, total - len(t)) for t in rc.tables]

    def can_grow(self, rc: RequestCache | None, num_new_tokens: int, keep_free: int = 0) -> bool:
        """Whether pages for ``num_new_tokens`` more tokens fit in every group, leaving
        ``keep_free`` pages (turingserve/kv/kv_manager.py:21-22).  ``rc`` None: a new request."""
        if rc is None:
            need = [-(-num_new_tokens // self.page_size)] * len(self.groups)
        else:
            need = self.pages_needed(rc, num_new_tokens)
        return all(g.allocator.num_free - n >= keep_free for g, n in zip(self.groups, need))

    def grow(self, rc: RequestCache, num_new_tokens: int) -> None:
        """Allocate pages so that positions < num_tokens + num_new_tokens have slots (all groups,
        or nothing and ``NoFreePages``)."""
        need = self.pages_needed(rc, num_new_tokens)
        for g, n in zip(self.groups, need):
            if g.allocator.num_free < n:
                raise NoFreePages(f"request {rc.request_id!r} needs {n} pages, {g.allocator.num_free} free")
        for g, n, table in zip(self.groups, need, rc.tables):
            for _ in range(n):
                table.append(g.allocator.allocate())

    def advance(self, rc: RequestCache, num_tokens: int) -> None:
        """``num_tokens`` more tokens are in the cache; give back pages a window has passed."""
        rc.num_tokens += num_tokens
        if self.groups and rc.num_tokens > len(rc.tables[0]) * self.page_size:
            raise RuntimeError("advance() beyond the pages that were grown")
        for gi, g in enumerate(self.groups):
            w = g.need.window
            if w is None:
                continue
            # the next query is at position >= num_tokens and sees keys >= num_tokens - w + 1
            first_needed = max(0, rc.num_tokens - w + 1)
            keep_from = first_needed // self.page_size
            table = rc.tables[gi]
            for p in range(rc.first_live_page[gi], min(keep_from, len(table))):
                if table[p] != 0:
                    g.allocator.free(table[p])
                    table[p] = 0
            rc.first_live_page[gi] = max(rc.first_live_page[gi], min(keep_from, len(table)))

    def release(self, rc: RequestCache) -> None:
        """Give back every page and the state slot (finish, abort or preemption)."""
        if self.live.get(rc.request_id) is not rc:
            raise ValueError(f"request {rc.request_id!r} released twice (or never admitted)")
        for g, table in zip(self.groups, rc.tables):
            for p in table:
                if p != 0:
                    g.allocator.free(p)
            table.clear()
        rc.num_tokens = 0
        rc.first_live_page = [0] * len(self.groups)
        del self.live[rc.request_id]
        self._free_slots.append(rc.slot)

    def slot_of(self, rc: RequestCache, group: int, pos: int) -> int:
        return rc.tables[group][pos // self.page_size] * self.page_size + pos % self.page_size

    # -- statistics / invariants ------------------------------------------------------------------
    def num_free(self, group: int = 0) -> int:
        return self.groups[group].allocator.num_free

    def min_free(self) -> int:
        return min((g.allocator.num_free for g in self.groups), default=0)

    def usage(self) -> float:
        if not self.groups:
            return 0.0
        return max(1.0 - g.allocator.num_free / g.allocator.num_usable for g in self.groups)

    def check(self) -> None:
        """No page lost, held twice or both free and held; slots consistent."""
        for gi, g in enumerate(self.groups):
            g.allocator.check()
            held = [p for rc in self.live.values() for p in rc.tables[gi] if p != 0]
            assert len(held) == len(set(held)), "a page is in two block tables"
            for p in held:
                assert g.allocator.is_held(p), f"page {p} is in a block table but free"
            assert len(held) + g.allocator.num_free == g.allocator.num_usable, "a page was lost"
        slots = [rc.slot for rc in self.live.values()]
        assert len(slots) == len(set(slots)), "a state slot is held twice"
        assert sorted(slots + self._free_slots) == list(range(self.max_requests)), "a state slot was lost"
