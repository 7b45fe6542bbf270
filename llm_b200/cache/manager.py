"""Host side of the cache: pages, block tables and state slots.

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


class _Group:
    def __init__(self, spec: GroupSpec):
        self.spec = spec
        self.free: List[int] = list(range(spec.num_pages - 1, -1, -1))   # pop() gives page 0 first
        self.tables: Dict[Hashable, List[int]] = {}      # logical page index -> physical page, -1 = given back
        self.first_live: Dict[Hashable, int] = {}        # first logical page still held

    def pages_for(self, length: int) -> int:
        return (length + self.spec.page_size - 1) // self.spec.page_size

    def dead_before(self, next_pos: int) -> int:
        """Logical pages below this index can no longer be seen by a token at next_pos or later."""
        if self.spec.kind != "window":
            return 0
        lowest_key = next_pos - self.spec.window + 1
        return max(0, lowest_key // self.spec.page_size)


class CacheManager:
    def __init__(self, groups: List[GroupSpec], max_requests: int, max_seq_len: int):
        if max_requests <= 0 or max_seq_len <= 0:
            raise CacheError("max_requests and max_seq_len must be positive")
        self._groups = [_Group(g) for g in groups]
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._slot: Dict[Hashable, int] = {}
        self._len: Dict[Hashable, int] = {}
        self.fresh_slots: List[int] = []      # admitted since the last take_fresh_slots(): state to be zeroed

    # ---- queries ----
    @property
    def num_groups(self) -> int:
        return len(self._groups)

    def group_spec(self, g: int) -> GroupSpec:
        return self._groups[g].spec

    def table_width(self, g: int) -> int:
        return self._groups[g].pages_for(self.max_seq_len)

    def num_free_pages(self, g: int) -> int:
        return len(self._groups[g].free)

    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def is_live(self, req: Hashable) -> bool:
        return req in self._slot

    def live_requests(self):
        return list(self._slot)

    def length(self, req: Hashable) -> int:
        return self._len[req]

    def slot(self, req: Hashable) -> int:
        return self._slot[req]

    def table(self, g: int, req: Hashable) -> List[int]:
        return self._groups[g].tables[req]

    def pages_needed(self, req: Optional[Hashable], n_new: int, length: Optional[int] = None) -> List[int]:
        """Per group, the pages that growing by n_new tokens takes from the free list, net of
        the window pages that the same call gives back first.  req None = a request not yet
        admitted (length 0 unless given)."""
        cur = self._len.get(req, 0) if length is None else length
        out = []
        for grp in self._groups:
            have_hi = grp.pages_for(cur)
            need_hi = grp.pages_for(cur + n_new)
            give_back = 0
            if grp.spec.kind == "window":
                first = grp.first_live.get(req, 0) if req in grp.tables else 0
                dead = min(grp.dead_before(cur), have_hi)
                give_back = max(0, dead - first)
            out.append(need_hi - have_hi - give_back)
        return out

    def can_extend(self, req: Optional[Hashable], n_new: int) -> bool:
        cur = self._len.get(req, 0)
        if cur + n_new > self.max_seq_len:
            return False
        return all(need <= len(grp.free) for need, grp in zip(self.pages_needed(req, n_new), self._groups))

    # ---- life cycle ----
    def admit(self, req: Hashable) -> int:
        """A new request takes a state slot; returns the slot."""
        if req in self._slot:
            raise CacheError(f"request {req!r} is already live")
        if not self._free_slots:
            raise CacheError(f"no request slot free ({self.max_requests} live)")
        slot = self._free_slots.pop()
        self._slot[req] = slot
        self._len[req] = 0
        for grp in self._groups:
            grp.tables[req] = []
            grp.first_live[req] = 0
        self.fresh_slots.append(slot)
        return slot

    def take_fresh_slots(self) -> List[int]:
        out, self.fresh_slots = self.fresh_slots, []
        return out

    def extend(self, req: Hashable, n_new: int) -> int:
        """The request is about to write n_new tokens: give back window pages that are out
        of sight, take the pages that the new tokens need, and return the position of the
        first new token (the reference's KV_Pool::append, kv/KV_pool.h:40-52)."""
        if req not in self._slot:
            raise CacheError(f"request {req!r} is not live")
        if n_new <= 0:
            raise CacheError("extend needs at least one token")
        cur = self._len[req]
        if cur + n_new > self.max_seq_len:
            raise CacheError(f"request {req!r}: {cur}+{n_new} tokens exceed max_seq_len {self.max_seq_len}")
        needs = self.pages_needed(req, n_new)
        for g, (need, grp) in enumerate(zip(needs, self._groups)):
            if need > len(grp.free):
                raise OutOfPages(f"group {g}: request {req!r} needs {need} pages, {len(grp.free)} free")
        for grp in self._groups:
            table = grp.tables[req]
            if grp.spec.kind == "window":
                dead = min(grp.dead_before(cur), len(table))
                for i in range(grp.first_live[req], dead):
                    grp.free.append(table[i])
                    table[i] = -1
                grp.first_live[req] = max(grp.first_live[req], dead)
            for _ in range(len(table), grp.pages_for(cur + n_new)):
                table.append(grp.free.pop())
        self._len[req] = cur + n_new
        return cur

    def release(self, req: Hashable) -> None:
        """The request ended: all its pages and its slot go back (kv/KV_pool.h:55-60)."""
        if req not in self._slot:
            raise CacheError(f"request {req!r} is not live (released twice?)")
        for grp in self._groups:
            table = grp.tables.pop(req)
            for i in range(grp.first_live.pop(req), len(table)):
                grp.free.append(table[i])
        self._free_slots.append(self._slot.pop(req))
        del self._len[req]

    def physical_slot(self, g: int, req: Hashable, pos: int) -> int:
        """page * page_size + offset of a held position (kv/KV_pool.h:76-79)."""
        grp = self._groups[g]
        page = grp.tables[req][pos // grp.spec.page_size]
        if page < 0:
            raise CacheError(f"position {pos} of request {req!r} was given back")
        return page * grp.spec.page_size + pos % grp.spec.page_size

    # ---- invariants, for tests ----
    def check(self) -> None:
        """No page lost, held twice or free twice; no slot lost or shared."""
        for g, grp in enumerate(self._groups):
            held = [p for req, t in grp.tables.items() for p in t[grp.first_live[req]:]]
            if any(p < 0 for p in held):
                raise CacheError(f"group {g}: a live table entry is marked as given back")
            both = held + grp.free
            if len(set(both)) != len(both):
                raise CacheError(f"group {g}: a page is held twice or free twice")
            if set(both) != set(range(grp.spec.num_pages)):
                raise CacheError(f"group {g}: pages lost: {set(range(grp.spec.num_pages)) - set(both)}")
            for req, t in grp.tables.items():
                if len(t) != grp.pages_for(self._len[req]):
                    raise CacheError(f"group {g}: table of {req!r} does not match its length")
        slots = list(self._slot.values()) + self._free_slots
        if sorted(slots) != list(range(self.max_requests)):
            raise CacheError("a request slot is lost or shared")
