"""Fixed-size pages and per-request state slots: the host-side allocators.

`PagePool` is the reference's allocator (`engine/src/paged.rs:65-144`): a stack
of free page ids and an in-use flag per page; running out is an error, a double
free or an out-of-range id is rejected instead of corrupting the free list.
`StateSlotPool` hands out one fixed-size slot per live request for mixers that
keep state of fixed size (the reference has none; the slot is there so such a
mixer needs no change to the engine).

Both are thin wrappers of one native type, a stack of ids (`csrc/host_cache.cpp`,
host code only), either one of their own or one that lives inside a cache manager.
"""
from __future__ import annotations

import ctypes

_lib = None


def native():
    """The native library of the cache manager, with its argument types set."""
    global _lib
    if _lib is not None:
        return _lib
    from ..ops import build
    lib = build.load("host_cache")
    vp, i, l, cp = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_char_p
    for name, res, args in [
            ("cb_stack_create", vp, [i]), ("cb_stack_destroy", None, [vp]),
            ("cb_stack_take", i, [vp]), ("cb_stack_give", i, [vp, i]),
            ("cb_stack_free", i, [vp]), ("cb_stack_in_use", i, [vp, i]),
            ("cb_cache_create", vp, [i, vp, vp, vp, i, vp, vp]), ("cb_cache_destroy", None, [vp]),
            ("cb_cache_stack", vp, [vp, i]), ("cb_cache_pages_for", l, [vp, i, l, l]),
            ("cb_cache_fits", i, [vp, l, l, i]), ("cb_cache_add", i, [vp, l, l, vp, cp, i]),
            ("cb_cache_extend", i, [vp, i, l, cp, i]), ("cb_cache_shrink", i, [vp, i, l]),
            ("cb_cache_remove", i, [vp, i]),
            ("cb_cache_step", i, [vp, i, vp, vp, l, vp, vp, vp, cp, i]),
            ("cb_cache_unstep", i, [vp, i, vp, vp]), ("cb_cache_is_live", i, [vp, i]),
            ("cb_cache_length", l, [vp, i]), ("cb_cache_table_len", i, [vp, i, i]),
            ("cb_cache_table_copy", None, [vp, i, i, vp]), ("cb_cache_held", i, [vp, i, i]),
            ("cb_cache_reserved", l, [vp, i]), ("cb_cache_row", vp, [vp, i, i]),
            ("cb_cache_poke", None, [vp, i, i, i, i]), ("cb_cache_check", i, [vp, vp, cp, i]),
            ("cb_cache_check_tables", i, [vp, vp, cp, i])]:
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


# result codes of the native calls
OK, PAGES_EXHAUSTED, SLOTS_EXHAUSTED, NOT_LIVE, TOO_LONG, ALIASED, DOUBLE_FREE, OUT_OF_RANGE, \
    BROKEN, BAD_ARGUMENT = range(10)


class CacheError(RuntimeError):
    pass


class PoolExhausted(CacheError):
    pass


class _IdStack:
    """A native stack of ids: its own (made and destroyed here) or a view of one that
    `keeper` owns."""

    def __init__(self, n: int, handle=None, keeper=None):
        self._lib = native()
        self._n = n
        self._keeper = keeper
        self._own = handle is None
        self._h = self._lib.cb_stack_create(n) if handle is None else handle
        if not self._h:
            raise ValueError("a pool needs a positive size")

    def __del__(self):
        if getattr(self, "_own", False) and self._h:
            self._lib.cb_stack_destroy(self._h)
            self._h = None

    def _free_count(self) -> int:
        return self._lib.cb_stack_free(self._h)

    def _take(self) -> int:
        return self._lib.cb_stack_take(self._h)

    def _give(self, i: int) -> int:
        return self._lib.cb_stack_give(self._h, int(i))


class PagePool(_IdStack):
    def __init__(self, n_pages: int, page_tokens: int, _handle=None, _keeper=None):
        if n_pages <= 0 or page_tokens <= 0:
            raise ValueError("a page pool needs a positive number of pages and tokens per page")
        super().__init__(n_pages, _handle, _keeper)
        self.n_pages = n_pages
        self.page_tokens = page_tokens

    @property
    def free_pages(self) -> int:
        return self._free_count()

    @property
    def used_pages(self) -> int:
        return self.n_pages - self._free_count()

    def alloc(self) -> int:
        page = self._take()
        if page < 0:
            raise PoolExhausted(f"kv page pool exhausted: all {self.n_pages} pages "
                                f"({self.n_pages * self.page_tokens} tokens) are in use")
        return page

    def release(self, page: int) -> None:
        code = self._give(page)
        if code == OUT_OF_RANGE:
            raise CacheError(f"page {page} out of range (pool has {self.n_pages} pages)")
        if code == DOUBLE_FREE:
            raise CacheError(f"double free of kv page {page}")

    def is_in_use(self, page: int) -> bool:
        if not 0 <= page < self.n_pages:
            raise IndexError(f"page {page} out of range (pool has {self.n_pages} pages)")
        return bool(self._lib.cb_stack_in_use(self._h, int(page)))


class StateSlotPool(_IdStack):
    def __init__(self, n_slots: int, _handle=None, _keeper=None):
        if n_slots <= 0:
            raise ValueError("a state slot pool needs at least one slot")
        super().__init__(n_slots, _handle, _keeper)
        self.n_slots = n_slots

    @property
    def free_slots(self) -> int:
        return self._free_count()

    def acquire(self) -> int:
        slot = self._take()
        if slot < 0:
            raise PoolExhausted(f"all {self.n_slots} request state slots are in use")
        return slot

    def release(self, slot: int) -> None:
        code = self._give(slot)
        if code == OUT_OF_RANGE:
            raise CacheError(f"state slot {slot} out of range ({self.n_slots} slots)")
        if code == DOUBLE_FREE:
            raise CacheError(f"double release of state slot {slot}")
