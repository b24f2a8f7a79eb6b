"""The cache manager: block tables per request and per cache group.

One `PagePool` per cache group (layers that keep all keys, layers that keep a
window of them, ... each have pages of their own), one block table per request
per group, one state slot per request.  Growth is all-or-nothing across groups
with rollback (`engine/src/paged.rs:199-217`); pages go back when a request
ends (`engine/src/runtime.rs:896-898`) or, in a windowed group, when the window
has passed them; freed pages are handed out again.  A logical reservation
ledger (`engine/src/prefill.rs:160-206`) lets a scheduler admit a request only
if its whole lifetime fits, so a running request never meets an empty pool.

Host-only: no device types here.  The block-table entry of a page that was
given back early is -1; kernels never read it because a windowed mixer starts
at the first key of its window.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from .pages import CacheError, PagePool, PoolExhausted, StateSlotPool

RELEASED = -1


@dataclass(frozen=True)
class GroupPolicy:
    page_tokens: int
    window: Optional[int] = None     # None: keep every token


@dataclass
class _Request:
    slot: int
    length: int = 0
    tables: List[List[int]] = field(default_factory=list)   # per group: logical block -> page
    first_live: List[int] = field(default_factory=list)     # per group: first block still held
    reserved: List[int] = field(default_factory=list)       # per group: pages reserved logically


class CacheManager:
    def __init__(self, policies: Sequence[GroupPolicy], pages_per_group: Sequence[int],
                 n_state_slots: int):
        if len(policies) != len(pages_per_group):
            raise ValueError("one page count per cache group is needed")
        self.policies = list(policies)
        self.pools = [PagePool(n, p.page_tokens) for p, n in zip(policies, pages_per_group)]
        self.slots = StateSlotPool(n_state_slots)
        self._requests: Dict[Hashable, _Request] = {}
        self._reserved = [0] * len(policies)

    # -- sizes ----------------------------------------------------------------

    def pages_for(self, group: int, n_tokens: int, max_step_tokens: Optional[int] = None) -> int:
        """Pages a request of `n_tokens` holds at most in `group` at any time."""
        pol = self.policies[group]
        full = -(-n_tokens // pol.page_tokens)
        if pol.window is None:
            return full
        step = n_tokens if max_step_tokens is None else max(1, min(max_step_tokens, n_tokens))
        # keys of the window before the step's first token, plus the step itself,
        # plus one page for misalignment at either end
        live = -(-(pol.window - 1 + step) // pol.page_tokens) + 1
        return min(full, live)

    # -- requests -------------------------------------------------------------

    def has(self, req) -> bool:
        return req in self._requests

    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    def length(self, req) -> int:
        return self._get(req).length

    def state_slot(self, req) -> int:
        return self._get(req).slot

    def can_reserve(self, lifetime_tokens: int, max_step_tokens: Optional[int] = None) -> bool:
        if self.slots.free_slots == 0:
            return False
        for g, pool in enumerate(self.pools):
            need = self.pages_for(g, lifetime_tokens, max_step_tokens)
            if need > pool.n_pages - self._reserved[g]:
                return False
        return True

    def fits_at_all(self, lifetime_tokens: int, max_step_tokens: Optional[int] = None) -> bool:
        return all(self.pages_for(g, lifetime_tokens, max_step_tokens) <= pool.n_pages
                   for g, pool in enumerate(self.pools))

    def add_request(self, req, lifetime_tokens: Optional[int] = None,
                    max_step_tokens: Optional[int] = None) -> int:
        """Registers a request, takes its state slot and, if `lifetime_tokens`
        is given, reserves that many tokens' pages logically in every group.
        Raises PoolExhausted (changing nothing) if slot or reservation fail."""
        if req in self._requests:
            raise CacheError(f"request {req!r} is already live")
        reserved = [0] * len(self.pools)
        if lifetime_tokens is not None:
            for g, pool in enumerate(self.pools):
                need = self.pages_for(g, lifetime_tokens, max_step_tokens)
                if need > pool.n_pages - self._reserved[g]:
                    raise PoolExhausted(
                        f"request {req!r} needs {need} pages in cache group {g}; "
                        f"{pool.n_pages - self._reserved[g]} of {pool.n_pages} are unreserved")
                reserved[g] = need
        slot = self.slots.acquire()
        for g, n in enumerate(reserved):
            self._reserved[g] += n
        self._requests[req] = _Request(slot=slot, tables=[[] for _ in self.pools],
                                       first_live=[0] * len(self.pools), reserved=reserved)
        return slot

    def extend(self, req, n_new: int) -> None:
        """Makes room for `n_new` more tokens of `req` in every group and commits
        them.  First gives back pages that the window has passed; then allocates,
        all or nothing: if any group runs out, the pages this call took go back
        and the request is as before."""
        if n_new <= 0:
            raise ValueError("extend needs a positive token count")
        r = self._get(req)
        self._release_passed(r)
        target = r.length + n_new
        taken: List[List[int]] = [[] for _ in self.pools]
        try:
            for g, pool in enumerate(self.pools):
                needed = -(-target // pool.page_tokens)
                while len(r.tables[g]) + len(taken[g]) < needed:
                    taken[g].append(pool.alloc())
        except PoolExhausted:
            for g, pages in enumerate(taken):
                for p in pages:
                    self.pools[g].release(p)
            raise
        for g, pages in enumerate(taken):
            r.tables[g].extend(pages)
        r.length = target

    def _release_passed(self, r: _Request) -> None:
        for g, pol in enumerate(self.policies):
            if pol.window is None:
                continue
            # the next token sits at position r.length and reads keys from
            # r.length - window + 1 on; blocks wholly below that are done
            first_needed = max(0, r.length - pol.window + 1)
            upto = min(first_needed // pol.page_tokens, len(r.tables[g]))
            for b in range(r.first_live[g], upto):
                self.pools[g].release(r.tables[g][b])
                r.tables[g][b] = RELEASED
            r.first_live[g] = max(r.first_live[g], upto)

    def remove_request(self, req) -> None:
        r = self._get(req)
        for g, table in enumerate(r.tables):
            # last page first: the pool is a stack, so the next request takes these pages in
            # the order this one held them, and runs of consecutive pages (which the attention
            # kernels fetch with one copy per tile instead of one per page) survive reuse
            for page in reversed(table):
                if page != RELEASED:
                    self.pools[g].release(page)
            self._reserved[g] -= r.reserved[g]
        self.slots.release(r.slot)
        del self._requests[req]

    # -- views ----------------------------------------------------------------

    def block_table(self, req, group: int) -> List[int]:
        return self._get(req).tables[group]

    def held_pages(self, req, group: int) -> int:
        return sum(1 for p in self._get(req).tables[group] if p != RELEASED)

    def free_pages(self, group: int) -> int:
        return self.pools[group].free_pages

    def reserved_pages(self, group: int) -> int:
        return self._reserved[group]

    def _get(self, req) -> _Request:
        try:
            return self._requests[req]
        except KeyError:
            raise CacheError(f"request {req!r} is not live") from None

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held."""
        for g, pool in enumerate(self.pools):
            seen = set()
            for req, r in self._requests.items():
                for page in r.tables[g]:
                    if page == RELEASED:
                        continue
                    if page in seen:
                        raise CacheError(f"page {page} of group {g} is held twice")
                    if not pool.is_in_use(page):
                        raise CacheError(f"page {page} of group {g} is held by {req!r} but free")
                    seen.add(page)
            if len(seen) != pool.used_pages:
                raise CacheError(f"group {g}: {pool.used_pages} pages in use but "
                                 f"{len(seen)} held by requests")
