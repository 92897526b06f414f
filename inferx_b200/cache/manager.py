"""Host-side cache bookkeeping: pages, block tables, per-request state slots.

The reference has one pool of blocks for all layers with a LIFO free list that
hands out block 0 first and treats a double free as an error
(src/core/kv_cache.cc:11-99), a host ``BlockTable`` per sequence
(include/inferx/core/kv_cache.h:158-186), and no per-request state.  Here:

* layers are put into *groups* by what they need kept (all tokens, or a window
  of them); each group has a page pool and a block table per request of its own,
  so a windowed group gives back pages that have fallen wholly behind the window
  while the full group keeps them;
* every request also holds one *state slot*, an index into tensors of fixed
  per-request size (recurrent state and the like); a slot handed out is reported
  as fresh once, so that whoever owns the tensors can zero it.

Nothing here touches a device: a block table is a list of page ids, with -1 for a
page that was given back.  The scheduler and the replay tool drive it; the
executor only reads it.
"""
from __future__ import annotations

from array import array
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence


class CacheError(RuntimeError):
    pass


class PagePool:
    """Page ids 0..n-1, LIFO free list (page 0 first), double free is an error."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._is_free = [True] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def allocate(self) -> Optional[int]:
        if not self._free:
            return None
        p = self._free.pop()
        self._is_free[p] = False
        return p

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise CacheError(f"page {page} is not in the pool of {self.num_pages}")
        if self._is_free[page]:
            raise CacheError(f"page {page} freed twice")
        self._is_free[page] = True
        self._free.append(page)

    def is_free(self, page: int) -> bool:
        return self._is_free[page]


@dataclass(frozen=True)
class CacheGroup:
    """Layers that keep the same span of tokens share page ids and block tables."""
    window: int = 0          # 0: every token; W: the last W tokens
    layers: tuple = ()       # indices of the layers whose caches live in this group


@dataclass
class _Request:
    slot: int
    length: int = 0                                  # tokens whose keys/values are in the cache
    tables: List["array"] = field(default_factory=list)     # per group: page id per page index
    first_live: List[int] = field(default_factory=list)     # per group: first page index still held


class CacheManager:
    def __init__(self, groups: Sequence[CacheGroup], pages_per_group, page_size: int,
                 max_slots: int):
        if page_size <= 0:
            raise CacheError("page_size must be positive")
        if max_slots <= 0:
            raise CacheError("max_slots must be positive")
        self.groups = list(groups)
        if isinstance(pages_per_group, int):
            pages_per_group = [pages_per_group] * len(self.groups)
        if len(pages_per_group) != len(self.groups):
            raise CacheError("one page count per group is required")
        self.page_size = page_size
        self.pools = [PagePool(n) for n in pages_per_group]
        self.max_slots = max_slots
        self._free_slots = list(range(max_slots - 1, -1, -1))
        self._fresh_slots: List[int] = []
        self._requests: Dict[Hashable, _Request] = {}

    # -- requests ------------------------------------------------------------
    def has(self, rid) -> bool:
        return rid in self._requests

    def live_requests(self):
        return list(self._requests)

    def free_slots(self) -> int:
        return len(self._free_slots)

    def free_pages(self, group: int = 0) -> int:
        return self.pools[group].free_count

    def open(self, rid) -> Optional[int]:
        """Give the request a state slot and empty tables; None if no slot is free."""
        if rid in self._requests:
            raise CacheError(f"request {rid!r} is already open")
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self._fresh_slots.append(slot)
        self._requests[rid] = _Request(slot=slot, tables=[array("i") for _ in self.groups],
                                       first_live=[0 for _ in self.groups])
        return slot

    def close(self, rid) -> None:
        """Give back every page and the slot."""
        r = self._req(rid)
        for g, table in enumerate(r.tables):
            for page in table:
                if page >= 0:
                    self.pools[g].release(page)
        self._free_slots.append(r.slot)
        if r.slot in self._fresh_slots:
            self._fresh_slots.remove(r.slot)
        del self._requests[rid]

    def take_fresh_slots(self) -> List[int]:
        """Slots handed out since the last call; their state must start from zero."""
        out, self._fresh_slots = self._fresh_slots, []
        return out

    def _req(self, rid) -> _Request:
        if rid not in self._requests:
            raise CacheError(f"request {rid!r} is not open")
        return self._requests[rid]

    def length(self, rid) -> int:
        return self._req(rid).length

    def slot(self, rid) -> int:
        return self._req(rid).slot

    def first_live(self, rid, group: int) -> int:
        """Index of the first page of the request this group still holds."""
        return self._req(rid).first_live[group]

    def table(self, rid, group: int) -> "array":
        """The request's block table in this group: an ``array('i')`` of page ids (it
        reads like a list and hands its memory to numpy without a copy)."""
        return self._req(rid).tables[group]

    def capacity(self, rid) -> int:
        """Tokens the request's pages can hold (the smallest over groups)."""
        r = self._req(rid)
        return min((len(t) * self.page_size for t in r.tables), default=1 << 62)

    def pages_held(self, rid, group: int) -> int:
        return sum(1 for p in self._req(rid).tables[group] if p >= 0)

    # -- growth ----------------------------------------------------------------
    def pages_missing(self, rid, new_len: int) -> List[int]:
        """Per group, pages that ``reserve(rid, new_len)`` would have to allocate."""
        r = self._req(rid)
        want = -(-new_len // self.page_size)
        return [max(0, want - len(t)) for t in r.tables]

    def reserve(self, rid, new_len: int) -> bool:
        """Make room for positions below ``new_len`` in every group.  All or
        nothing: on a shortage in any group, whatever this call took is given
        back and False is returned."""
        r = self._req(rid)
        want = -(-new_len // self.page_size)
        taken = []
        for g, table in enumerate(r.tables):
            while len(table) < want:
                page = self.pools[g].allocate()
                if page is None:
                    for gg, _ in reversed(taken):
                        self.pools[gg].release(r.tables[gg].pop())
                    return False
                table.append(page)
                taken.append((g, page))
        return True

    def advance(self, rid, n_tokens: int) -> None:
        """``n_tokens`` more tokens are in the cache; windowed groups give back
        the pages no later query can see."""
        r = self._req(rid)
        new_len = r.length + n_tokens
        if new_len > self.capacity(rid):
            raise CacheError(
                f"request {rid!r}: {new_len} tokens exceed the reserved capacity "
                f"{self.capacity(rid)}")
        r.length = new_len
        for g, grp in enumerate(self.groups):
            if grp.window <= 0:
                continue
            # the next query sits at position >= new_len and sees keys from
            # new_len - window + 1 on: a page whose last position is below that is dead
            first_needed = new_len - grp.window + 1
            table = r.tables[g]
            i = r.first_live[g]
            while i < len(table) and (i + 1) * self.page_size <= first_needed:
                if table[i] >= 0:
                    self.pools[g].release(table[i])
                    table[i] = -1
                i += 1
            r.first_live[g] = i

    # -- checks ----------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, held twice or both free and held; slots likewise."""
        for g, pool in enumerate(self.pools):
            held = []
            for rid, r in self._requests.items():
                held += [p for p in r.tables[g] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a page is held twice")
            for p in held:
                if pool.is_free(p):
                    raise CacheError(f"group {g}: page {p} is both free and held")
            if len(held) + pool.free_count != pool.num_pages:
                raise CacheError(
                    f"group {g}: {pool.num_pages - len(held) - pool.free_count} pages lost")
            if len(set(pool._free)) != len(pool._free):
                raise CacheError(f"group {g}: a page is on the free list twice")
        slots = [r.slot for r in self._requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots):
            raise CacheError("a state slot is held twice or both free and held")
        if len(slots) + len(self._free_slots) != self.max_slots:
            raise CacheError("a state slot was lost")


def is_paged_need(need) -> bool:
    """A need kept per token in pages (it says how long tokens are kept and how wide a
    token's record is), as opposed to state of fixed size per request."""
    return hasattr(need, "window") and hasattr(need, "kv_heads") and hasattr(need, "head_dim")


def groups_for(cache_needs_per_layer) -> List[CacheGroup]:
    """Group layers by the span of tokens their paged needs keep.

    ``cache_needs_per_layer[i]`` is the list of needs of layer ``i``'s mixer.  The span
    alone decides the group: a page is a span of tokens, so layers whose records differ
    in shape or number of entries can share page numbers and block tables."""
    by_window: Dict[int, List[int]] = {}
    for i, needs in enumerate(cache_needs_per_layer):
        for need in needs:
            if is_paged_need(need) and i not in by_window.setdefault(int(need.window), []):
                by_window[int(need.window)].append(i)
    return [CacheGroup(window=w, layers=tuple(ls)) for w, ls in sorted(by_window.items())]
