"""Fixed-size pages and per-request state slots: the host-side allocators.

`PagePool` is the reference's allocator (`engine/src/paged.rs:65-144`): a stack
of free page ids and an in-use flag per page; running out is an error, a double
free or an out-of-range id is rejected instead of corrupting the free list.
`StateSlotPool` hands out one fixed-size slot per live request for mixers that
keep state of fixed size (the reference has none; the slot is there so such a
mixer needs no change to the engine).
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    pass


class PoolExhausted(CacheError):
    pass


class PagePool:
    def __init__(self, n_pages: int, page_tokens: int):
        if n_pages <= 0 or page_tokens <= 0:
            raise ValueError("a page pool needs a positive number of pages and tokens per page")
        self.n_pages = n_pages
        self.page_tokens = page_tokens
        # Reversed so that the first allocation is page 0 (paged.rs:75-77).
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._in_use = [False] * n_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.n_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise PoolExhausted(f"kv page pool exhausted: all {self.n_pages} pages "
                                f"({self.n_pages * self.page_tokens} tokens) are in use")
        page = self._free.pop()
        self._in_use[page] = True
        return page

    def release(self, page: int) -> None:
        if not 0 <= page < self.n_pages:
            raise CacheError(f"page {page} out of range (pool has {self.n_pages} pages)")
        if not self._in_use[page]:
            raise CacheError(f"double free of kv page {page}")
        self._in_use[page] = False
        self._free.append(page)

    def is_in_use(self, page: int) -> bool:
        return self._in_use[page]


class StateSlotPool:
    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise ValueError("a state slot pool needs at least one slot")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._in_use = [False] * n_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise PoolExhausted(f"all {self.n_slots} request state slots are in use")
        slot = self._free.pop()
        self._in_use[slot] = True
        return slot

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.n_slots:
            raise CacheError(f"state slot {slot} out of range ({self.n_slots} slots)")
        if not self._in_use[slot]:
            raise CacheError(f"double release of state slot {slot}")
        self._in_use[slot] = False
        self._free.append(slot)
