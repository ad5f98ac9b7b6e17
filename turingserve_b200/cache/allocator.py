"""Page allocator: a FIFO free list over page ids 1..N-1; page 0 is the null page that padded
block-table entries point at and is never handed out
(turingserve/kv/block_allocator.py:16-62: free deque, null block 0, NoFreeBlocks).
"""

from __future__ import annotations

from collections import deque


class NoFreePages(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int) -> None:
        if num_pages < 2:
            raise ValueError("a pool needs at least 2 pages (page 0 is the null page)")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(1, num_pages))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_usable(self) -> int:
        return self.num_pages - 1

    def allocate(self) -> int:
        if not self._free:
            raise NoFreePages("no free pages")
        page = self._free.popleft()
        self._held[page] = True
        return page

    def free(self, page: int) -> None:
        if page <= 0 or page >= self.num_pages:
            raise ValueError(f"page {page} is not an allocatable page")
        if not self._held[page]:
            raise ValueError(f"page {page} freed twice (or never allocated)")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]

    def shuffle_free_list(self, rng) -> None:
        """Test hook: randomise the order in which free pages are handed out."""
        pages = list(self._free)
        rng.shuffle(pages)
        self._free = deque(pages)

    def check(self) -> None:
        free = list(self._free)
        assert len(free) == len(set(free)), "a page is on the free list twice"
        assert 0 not in free, "the null page is on the free list"
        for p in free:
            assert not self._held[p], f"page {p} is both free and held"
        assert sum(self._held) + len(free) == self.num_pages - 1, "a page was lost"
