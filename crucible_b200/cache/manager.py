"""The cache manager: block tables per request and per cache group.

One page pool per cache group (layers that keep all keys, layers that keep a
window of them, ... each have pages of their own), one block table per request
per group, one state slot per request.  Growth is all-or-nothing across groups
with rollback (`engine/src/paged.rs:199-217`); pages go back when a request
ends (`engine/src/runtime.rs:896-898`) or, in a windowed group, when the window
has passed them; freed pages are handed out again.  A logical reservation
ledger (`engine/src/prefill.rs:160-206`) lets a scheduler admit a request only
if its whole lifetime fits, so a running request never meets an empty pool.

The bookkeeping itself is native host code (`csrc/host_cache.cpp`), as the
reference's is (`engine/src/paged.rs`); this class gives it the requests' own
names (any hashable) and Python's errors.  Host-only: no device types here.  A
block-table entry whose page was given back early reads `RELEASED`; in the row
that goes to the device (kept if `table_strides` is given) it names the null
page instead, so a kernel that loads whole tiles reads zeros there.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from . import pages as _pages
from .pages import CacheError, PagePool, PoolExhausted, StateSlotPool

RELEASED = -1


@dataclass(frozen=True)
class GroupPolicy:
    page_tokens: int
    window: Optional[int] = None     # None: keep every token


def _opt(value: Optional[int]) -> int:
    return -1 if value is None else int(value)


class CacheManager:
    def __init__(self, policies: Sequence[GroupPolicy], pages_per_group: Sequence[int],
                 n_state_slots: int, table_strides: Optional[Sequence[int]] = None,
                 null_pages: Optional[Sequence[int]] = None):
        """`table_strides`: ints of a request's device table row per group; with it the
        manager keeps every live request's row up to date at a fixed address
        (`step_raw` hands the addresses out) and refuses a request whose table would
        outgrow it.  `null_pages`: what such a row holds for a page given back early."""
        if len(policies) != len(pages_per_group):
            raise ValueError("one page count per cache group is needed")
        for p, n in zip(policies, pages_per_group):
            if n <= 0 or p.page_tokens <= 0:
                raise ValueError("a page pool needs a positive number of pages and tokens per page")
        if n_state_slots <= 0:
            raise ValueError("a state slot pool needs at least one slot")
        self.policies = list(policies)
        self._lib = lib = _pages.native()
        n = len(self.policies)
        arr = lambda values: (ctypes.c_int32 * max(1, n))(*values)
        self._h = lib.cb_cache_create(
            n, arr(p.page_tokens for p in self.policies), arr(_opt(p.window) for p in self.policies),
            arr(pages_per_group), n_state_slots,
            arr(table_strides) if table_strides is not None else None,
            arr(null_pages) if null_pages is not None else None)
        if not self._h:
            raise ValueError("the cache manager's sizes must be positive")
        self.table_strides = tuple(table_strides) if table_strides is not None else None
        self.pools = [PagePool(count, p.page_tokens, _handle=lib.cb_cache_stack(self._h, g),
                               _keeper=self)
                      for g, (p, count) in enumerate(zip(self.policies, pages_per_group))]
        self.slots = StateSlotPool(n_state_slots, _handle=lib.cb_cache_stack(self._h, -1),
                                   _keeper=self)
        self._slot_of: Dict[Hashable, int] = {}
        self._request_in = [None] * n_state_slots
        self._err = ctypes.create_string_buffer(256)
        self._info = (ctypes.c_int32 * 4)()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.cb_cache_destroy(self._h)
            self._h = None

    def _message(self) -> str:
        return self._err.value.decode(errors="replace")

    def _raise(self, code: int, req=None) -> None:
        who = "" if req is None else f"request {req!r}: "
        kind = PoolExhausted if code in (_pages.PAGES_EXHAUSTED, _pages.SLOTS_EXHAUSTED) else CacheError
        raise kind(who + self._message())

    # -- sizes ----------------------------------------------------------------

    def pages_for(self, group: int, n_tokens: int, max_step_tokens: Optional[int] = None) -> int:
        """Pages a request of `n_tokens` holds at most in `group` at any time."""
        return self._lib.cb_cache_pages_for(self._h, group, n_tokens, _opt(max_step_tokens))

    # -- requests -------------------------------------------------------------

    def has(self, req) -> bool:
        return req in self._slot_of

    def live_requests(self) -> List[Hashable]:
        return list(self._slot_of)

    def length(self, req) -> int:
        return self._lib.cb_cache_length(self._h, self._get(req))

    def state_slot(self, req) -> int:
        return self._get(req)

    def request_in_slot(self, slot: int):
        return self._request_in[slot]

    def can_reserve(self, lifetime_tokens: int, max_step_tokens: Optional[int] = None) -> bool:
        return bool(self._lib.cb_cache_fits(self._h, lifetime_tokens, _opt(max_step_tokens), 0))

    def fits_at_all(self, lifetime_tokens: int, max_step_tokens: Optional[int] = None) -> bool:
        return bool(self._lib.cb_cache_fits(self._h, lifetime_tokens, _opt(max_step_tokens), 1))

    def add_request(self, req, lifetime_tokens: Optional[int] = None,
                    max_step_tokens: Optional[int] = None) -> int:
        """Registers a request, takes its state slot and, if `lifetime_tokens`
        is given, reserves that many tokens' pages logically in every group.
        Raises PoolExhausted (changing nothing) if slot or reservation fail."""
        if req in self._slot_of:
            raise CacheError(f"request {req!r} is already live")
        slot = ctypes.c_int32(-1)
        code = self._lib.cb_cache_add(self._h, _opt(lifetime_tokens), _opt(max_step_tokens),
                                      ctypes.byref(slot), self._err, 256)
        if code:
            self._raise(code, req)
        self._slot_of[req] = slot.value
        self._request_in[slot.value] = req
        return slot.value

    def extend(self, req, n_new: int) -> None:
        """Makes room for `n_new` more tokens of `req` in every group and commits
        them.  First gives back pages that the window has passed; then allocates,
        all or nothing: if any group runs out, the pages this call took go back
        and the request is as before."""
        if n_new <= 0:
            raise ValueError("extend needs a positive token count")
        code = self._lib.cb_cache_extend(self._h, self._get(req), n_new, self._err, 256)
        if code:
            self._raise(code, req)

    def shrink(self, req, n: int) -> None:
        """Takes the request's last `n` tokens back, with the pages only they needed."""
        code = self._lib.cb_cache_shrink(self._h, self._get(req), n)
        if code:
            raise CacheError(f"request {req!r}: its last {n} tokens could not be taken back "
                             f"(code {code})")

    def remove_request(self, req) -> None:
        slot = self._get(req)
        code = self._lib.cb_cache_remove(self._h, slot)
        del self._slot_of[req]
        self._request_in[slot] = None
        if code:
            raise CacheError(f"request {req!r}: a page or its slot could not be given back "
                             f"(double free or out of range, code {code})")

    # -- a whole step at once -----------------------------------------------------

    def step_raw(self, n_req: int, slots_ptr: int, counts_ptr: int, max_tokens: Optional[int],
                 first_pos_ptr: int, rows) -> int:
        """Every request of a step (int32 arrays of state slots and token counts, by
        address) grows by its count, or none does.  Fills `first_pos` (what each held
        before) and `rows` (a ctypes array of n_groups * n_req addresses, group-major, of
        the device table rows; or None).  Returns 0, or the native code; then
        `failed_entry()` is the index of the request at fault and `raise_for(code, req)`
        raises its error."""
        return self._lib.cb_cache_step(self._h, n_req, slots_ptr, counts_ptr, _opt(max_tokens),
                                       first_pos_ptr, rows, ctypes.byref(self._info, 0), self._err,
                                       256)

    def failed_entry(self) -> int:
        return self._info[0]

    def raise_for(self, code: int, req=None) -> None:
        self._raise(code, req)

    def unstep_raw(self, n_req: int, slots_ptr: int, counts_ptr: int) -> None:
        """Undoes a step that `step_raw` accepted."""
        code = self._lib.cb_cache_unstep(self._h, n_req, slots_ptr, counts_ptr)
        if code:
            raise CacheError(f"a step could not be undone (code {code})")

    def extend_step(self, requests: Sequence[Hashable], counts: Sequence[int],
                    max_tokens: Optional[int] = None) -> List[int]:
        """`step_raw` for callers with lists: returns what each request held before."""
        ints = np.array([[self._get(r) for r in requests], list(counts)], dtype=np.int32)
        first = np.zeros(len(requests), dtype=np.int32)
        code = self.step_raw(len(requests), ints[0].ctypes.data, ints[1].ctypes.data, max_tokens,
                             first.ctypes.data, None)
        if code:
            self._raise(code, requests[self.failed_entry()])
        return first.tolist()

    # -- views ----------------------------------------------------------------

    def block_table(self, req, group: int) -> List[int]:
        """A copy of the request's table of `group`: logical block -> page, or RELEASED."""
        slot = self._get(req)
        n = self._lib.cb_cache_table_len(self._h, slot, group)
        out = (ctypes.c_int32 * max(1, n))()
        self._lib.cb_cache_table_copy(self._h, slot, group, out)
        return list(out[:n])

    def table_row(self, req, group: int) -> np.ndarray:
        """The request's table as it goes to the device (a copy): padded with zeros to the
        stride, the null page where a page was given back early."""
        if self.table_strides is None:
            raise CacheError("this cache manager keeps no device table rows")
        ptr = self._lib.cb_cache_row(self._h, self._get(req), group)
        stride = self.table_strides[group]
        return np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctypes.c_int32)),
                                     shape=(stride,)).copy()

    def held_pages(self, req, group: int) -> int:
        return self._lib.cb_cache_held(self._h, self._get(req), group)

    def free_pages(self, group: int) -> int:
        return self.pools[group].free_pages

    def reserved_pages(self, group: int) -> int:
        return self._lib.cb_cache_reserved(self._h, group)

    def _get(self, req) -> int:
        try:
            return self._slot_of[req]
        except KeyError:
            raise CacheError(f"request {req!r} is not live") from None

    def _poke(self, req, group: int, block: int, page: int) -> None:
        """For tests of the checks: changes a table entry behind the manager's back."""
        if not 0 <= block < self._lib.cb_cache_table_len(self._h, self._get(req), group):
            raise IndexError("no such block")
        self._lib.cb_cache_poke(self._h, self._get(req), group, block, page)

    def check_invariants(self) -> None:
        """No page lost, held twice or free while held."""
        code = self._lib.cb_cache_check(self._h, self._info, self._err, 256)
        if code:
            slot = self._info[2]
            who = f" (request {self._request_in[slot]!r})" if 0 <= slot < len(self._request_in) else ""
            raise CacheError(self._message() + who)
        if sorted(self._slot_of.values()) != [s for s, r in enumerate(self._request_in) if r is not None]:
            raise CacheError("the requests' names and their slots do not agree")

    def check_tables(self) -> None:
        """The tables by themselves, every entry: each page inside its pool, and none named
        by two requests or twice by one.  Growth checks this for the pages it adds; this is
        the whole check, for tests and for a host that suspects its allocator."""
        code = self._lib.cb_cache_check_tables(self._h, self._info, self._err, 256)
        if code:
            a, b = self._info[2], self._info[3]
            who = f": request {self._request_in[a]!r}"
            if 0 <= b < len(self._request_in):
                who += f" and request {self._request_in[b]!r}"
            raise CacheError(self._message() + who)
