"""Host side of the cache: pages, block tables and state slots.

The bookkeeping itself is native (csrc/host/page_pool.cpp, plain C++ behind a C interface, as the
reference's pool is C++); this module holds the group descriptions, the exceptions and the class
that maps the caller's request ids to the pool's slots.

Like the reference's KV_Pool (kv/KV_pool.h:13-102) this keeps, per request, the
list of physical pages that hold its tokens, hands pages out from a LIFO free list
when a request grows and takes them back when it ends.  Unlike it, the pool is
split into groups: layers whose needs differ (every past key, or a window of them)
have pages and tables of their own, and a window group gives a page back as soon
as every later token's window has passed it.  Page size is a parameter, not the
constant 16 of kv/KV_Layout.h:2, and contracts are checked, not asserted.

Beside the pages there is one state slot per live request (the row id that the
reference already uses to index its tables, kv/KV_pool.h:31-37), for parts that
keep per-request state of fixed size.

All device work of an engine runs in order on one stream, so a page may be handed
to another request as soon as the host has freed it: any kernel that still reads
it was launched before the kernel that will overwrite it.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional


class CacheError(RuntimeError):
    """A contract of the cache manager was broken by its caller."""


class OutOfPages(CacheError):
    """A request asked for more pages than its group has free."""


@dataclass(frozen=True)
class GroupSpec:
    kind: str                      # "full" | "window"
    page_size: int
    num_pages: int
    window: Optional[int] = None   # tokens visible to a query, itself included

    def __post_init__(self):
        if self.kind not in ("full", "window"):
            raise CacheError(f"unknown cache group kind '{self.kind}'")
        if self.kind == "window" and not (self.window and self.window > 0):
            raise CacheError("a window group needs a positive window")
        if self.page_size <= 0 or self.num_pages < 0:
            raise CacheError("page_size must be positive and num_pages non-negative")


_KINDS = {"full": 0, "window": 1}
_OUT_OF_PAGES = -2


_NAMED_KEYS = 1 << 62       # keys of ids that are not integers start here


class CacheManager:
    """Requests by their caller's ids on top of the native page pool (csrc/host/page_pool.cpp),
    which does the bookkeeping (pages, tables, window give-back, slots, the live requests and
    their slots, invariants) and knows a request by a 64-bit key: an integer id is its own key,
    any other hashable id gets one here.  This class turns the pool's error codes into
    exceptions.  The native scheduler works on the same pool, so a request that it releases is
    gone here too."""

    def __init__(self, groups: List[GroupSpec], max_requests: int, max_seq_len: int):
        if max_requests <= 0 or max_seq_len <= 0:
            raise CacheError("max_requests and max_seq_len must be positive")
        from ..csrc.build import load_host
        self._lib = lib = load_host()
        lib.llmh_pool_create.restype = ctypes.c_void_p
        lib.llmh_pool_error.restype = ctypes.c_char_p
        lib.llmh_pool_table.restype = ctypes.POINTER(ctypes.c_int)
        self._specs = list(groups)
        n = len(groups)
        arr = lambda vals: (ctypes.c_int * max(n, 1))(*vals)
        self._pool = lib.llmh_pool_create(
            n, arr([_KINDS[g.kind] for g in groups]), arr([g.page_size for g in groups]),
            arr([g.num_pages for g in groups]), arr([g.window or 0 for g in groups]), max_requests, max_seq_len)
        if not self._pool:
            raise CacheError("the page pool refused these groups")
        self._pool = ctypes.c_void_p(self._pool)
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        lib.llmh_pool_admit.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        lib.llmh_pool_slot.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        self._named: Dict[Hashable, int] = {}          # ids that are not integers -> keys
        self._names: Dict[int, Hashable] = {}
        self._next_named = 0
        self._keys = (ctypes.c_longlong * max_requests)()
        self._needs = (ctypes.c_int * max(n, 1))()
        self._fresh = (ctypes.c_int * max_requests)()

    def __del__(self):
        pool, self._pool = getattr(self, "_pool", None), None
        if pool:
            self._lib.llmh_pool_destroy(pool)

    def _fail(self, code: int):
        msg = self._lib.llmh_pool_error(self._pool).decode("utf-8", "replace")
        raise (OutOfPages if code == _OUT_OF_PAGES else CacheError)(msg)

    @property
    def native(self):
        """(library, pool handle) for callers that hand the pool to other native routines."""
        return self._lib, self._pool

    # ---- queries ----
    @property
    def num_groups(self) -> int:
        return len(self._specs)

    def group_spec(self, g: int) -> GroupSpec:
        return self._specs[g]

    def table_width(self, g: int) -> int:
        return self._lib.llmh_pool_table_width(self._pool, g)

    def num_free_pages(self, g: int) -> int:
        return self._lib.llmh_pool_free_pages(self._pool, g)

    def num_free_slots(self) -> int:
        return self._lib.llmh_pool_free_slots(self._pool)

    def key(self, req: Hashable, create: bool = False):
        """The 64-bit key under which the pool knows the request; None for an id that is not an
        integer and has no key yet (unless create)."""
        if isinstance(req, int) and not isinstance(req, bool):
            if not -_NAMED_KEYS <= req < _NAMED_KEYS:
                raise CacheError(f"request id {req} is out of range")
            return req
        k = self._named.get(req)
        if k is None and create:
            k = self._named[req] = _NAMED_KEYS + self._next_named
            self._next_named += 1
            self._names[k] = req
        return k

    def _slot_or_none(self, req: Hashable) -> int:
        k = self.key(req)
        return -1 if k is None else self._lib.llmh_pool_slot(self._pool, k)

    def is_live(self, req: Hashable) -> bool:
        return self._slot_or_none(req) >= 0

    def live_requests(self):
        n = self._lib.llmh_pool_live_keys(self._pool, self._keys, self.max_requests)
        return [self._names.get(k, k) for k in self._keys[:n]]

    def length(self, req: Hashable) -> int:
        return self._lib.llmh_pool_length(self._pool, self.slot(req))

    def slot(self, req: Hashable) -> int:
        slot = self._slot_or_none(req)
        if slot < 0:
            raise CacheError(f"request {req!r} is not live")
        return slot

    def table(self, g: int, req: Hashable) -> List[int]:
        """The request's logical pages in group g (-1 = given back)."""
        n, first = ctypes.c_int(), ctypes.c_int()
        row = self._lib.llmh_pool_table(self._pool, g, self.slot(req), ctypes.byref(n), ctypes.byref(first))
        return [row[i] for i in range(n.value)]

    def pages_needed(self, req: Optional[Hashable], n_new: int, length: Optional[int] = None) -> List[int]:
        """Per group, the pages that growing by n_new tokens takes from the free list, net of
        the window pages that the same call gives back first.  req None = a request not yet
        admitted (length 0 unless given)."""
        slot = self._slot_or_none(req) if req is not None else -1
        rc = self._lib.llmh_pool_pages_needed(self._pool, slot, -1 if length is None else length, n_new, self._needs)
        if rc < 0:
            self._fail(rc)
        return list(self._needs[:len(self._specs)])

    def can_extend(self, req: Optional[Hashable], n_new: int) -> bool:
        cur = self.length(req) if req is not None and self.is_live(req) else 0
        if cur + n_new > self.max_seq_len:
            return False
        return all(need <= self.num_free_pages(g) for g, need in enumerate(self.pages_needed(req, n_new)))

    # ---- life cycle ----
    def admit(self, req: Hashable) -> int:
        """A new request takes a state slot; returns the slot."""
        slot = self._lib.llmh_pool_admit(self._pool, self.key(req, create=True))
        if slot < 0:
            self._fail(slot)
        return slot

    def begin_step(self, reqs, counts, slots, starts) -> None:
        """The start of a step, all or nothing: request reqs[b] (admitted here if it is new) grows
        by counts[b] tokens; slots[b] and starts[b] receive its slot and the position of its first
        new token.  counts, slots and starts are int32 numpy arrays.  Nothing has moved if it
        raises: CacheError (no request slot, or max_seq_len) or OutOfPages."""
        n = len(reqs)
        keys = (ctypes.c_longlong * max(n, 1))(*[self.key(r, create=True) for r in reqs])
        bad = ctypes.c_int()
        ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        rc = self._lib.llmh_pool_begin_step(self._pool, n, keys, ptr(counts), ptr(slots), ptr(starts), ctypes.byref(bad))
        if rc < 0:
            msg = self._lib.llmh_pool_error(self._pool).decode("utf-8", "replace")
            if rc != _OUT_OF_PAGES and bad.value >= 0:
                msg = f"request {reqs[bad.value]!r}: {msg}"
            raise (OutOfPages if rc == _OUT_OF_PAGES else CacheError)(msg)

    def take_fresh_slots(self) -> List[int]:
        """Slots admitted since the last call: their state is to be zeroed."""
        n = self._lib.llmh_pool_take_fresh(self._pool, self._fresh, self.max_requests)
        return list(self._fresh[:n])

    def log_freed_pages(self, on: bool = True) -> None:
        """Debug aid: remember every page that goes back to a free list until take_freed_pages
        collects it."""
        self._lib.llmh_pool_log_freed(self._pool, int(on))

    def take_freed_pages(self, g: int) -> List[int]:
        """Pages of group g that were given back since the last call (after log_freed_pages)."""
        out: List[int] = []
        buf = (ctypes.c_int * 256)()
        while True:
            n = self._lib.llmh_pool_take_freed(self._pool, g, buf, 256)
            out.extend(buf[:n])
            if n < 256:
                return out

    def extend(self, req: Hashable, n_new: int) -> int:
        """The request is about to write n_new tokens: give back window pages that are out
        of sight, take the pages that the new tokens need, and return the position of the
        first new token (the reference's KV_Pool::append, kv/KV_pool.h:40-52)."""
        start = self._lib.llmh_pool_extend(self._pool, self.slot(req), n_new)
        if start < 0:
            self._fail(start)
        return start

    def release(self, req: Hashable) -> None:
        """The request ended: all its pages and its slot go back (kv/KV_pool.h:55-60)."""
        slot = self._slot_or_none(req)
        if slot < 0:
            raise CacheError(f"request {req!r} is not live (released twice?)")
        rc = self._lib.llmh_pool_release(self._pool, slot)
        if rc < 0:
            self._fail(rc)
        k = self._named.pop(req, None) if not isinstance(req, int) or isinstance(req, bool) else None
        if k is not None:
            del self._names[k]

    def physical_slot(self, g: int, req: Hashable, pos: int) -> int:
        """page * page_size + offset of a held position (kv/KV_pool.h:76-79)."""
        ps = self._specs[g].page_size
        table = self.table(g, req)
        page = table[pos // ps]
        if page < 0:
            raise CacheError(f"position {pos} of request {req!r} was given back")
        return page * ps + pos % ps

    # ---- invariants, for tests ----
    def check(self) -> None:
        """No page lost, held twice or free twice; no slot lost or shared."""
        rc = self._lib.llmh_pool_check(self._pool)
        if rc < 0:
            self._fail(rc)
