"""The cache manager: keys and values in pages with a block table per request, and
slots for per-request state of fixed size.

Layers are put into groups by what they need: layers that keep every key of a
request form one group, layers that only ever read a window of the last W keys
form another (one per distinct W and shape).  A group has a page pool of its own,
a device tensor [layers of the group, 2 (k, v), pages, kv heads, page_size,
head_dim], and a block table per request, so one page id addresses the same slot
in every layer of its group (as in the reference's pool,
backend/model.cu:41, 1096-1097) and groups never compete for pages.

Protocol, as in the reference (engine/kv/kv.go:54-74; engine/engine.go:160-168):
``reserve(req, n)`` before a step makes the tables cover n more tokens,
``commit(req, n)`` after it advances the length, ``close(req)`` gives everything
back.  Unlike the reference, a reservation is all-or-nothing over all groups: when
pages run out nothing is held that was not held before.  A window group gives a
page back as soon as the window has passed it (at commit); its table keeps -1 in
that place.  Pages are handed out last-freed-first (kv.go:29-40), so reuse is
immediate.

Beside the pages, every request holds one state slot.  A mixer with per-request
state of fixed size (``StateNeed``) gets a tensor [max_requests, *shape] per layer,
and the slot's rows are zeroed when a request opens.  This architecture has no
such mixer; the slots are handed out and taken back all the same.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..parts.context import LayerCache
from ..parts.spec import PagedKVNeed, StateNeed


class OutOfPages(RuntimeError):
    """A reservation could not be met; nothing was taken."""


class CacheError(RuntimeError):
    """Misuse of the manager (double free, foreign page, closed request)."""


class IdPool:
    """A fixed set of ids 0..n-1 with a LIFO free list; low ids go out first."""

    def __init__(self, n: int, what: str = "page"):
        if n <= 0:
            raise ValueError(f"a pool needs at least one {what}, got {n}")
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))
        self._held = [False] * n
        self.high_water = 0

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.n - len(self._free)

    def take(self, count: int) -> List[int]:
        if count > len(self._free):
            raise OutOfPages(f"out of {self.what}s: {count} wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(count)]
        for i in out:
            self._held[i] = True
        self.high_water = max(self.high_water, self.used_count)
        return out

    def give(self, ids: Sequence[int]) -> None:
        for i in ids:
            if not (0 <= i < self.n):
                raise CacheError(f"{self.what} {i} does not belong to this pool of {self.n}")
            if not self._held[i]:
                raise CacheError(f"{self.what} {i} is freed twice")
            self._held[i] = False
            self._free.append(i)


@dataclass
class CacheGroup:
    index: int
    need: PagedKVNeed
    slots: List[int]           # cache slots (layer calls) that live in this group
    page_size: int
    pool: IdPool
    storage: Optional[torch.Tensor] = None   # [len(slots), 2, pages, kv heads, page_size, head_dim]

    @property
    def window(self) -> Optional[int]:
        return self.need.window


@dataclass
class RequestCache:
    """One live request's hold on the cache."""
    rid: int
    state_slot: int
    length: int = 0                                  # tokens committed
    tables: List[List[int]] = field(default_factory=list)   # per group, logical page -> page id or -1
    closed: bool = False

    def pages_held(self) -> int:
        return sum(1 for t in self.tables for p in t if p >= 0)


class CacheManager:
    def __init__(self, needs: Sequence, page_size: int, num_pages: int, max_requests: int,
                 dtype: torch.dtype = torch.float32, device="cpu", allocate: bool = True):
        """``needs[i]`` is what cache slot i asks for: None, a PagedKVNeed, a
        StateNeed, or a list of them.  ``num_pages`` is the size of every group's pool."""
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = torch.device(device)
        self.groups: List[CacheGroup] = []
        self.slot_group: Dict[int, int] = {}       # cache slot -> group index
        self.slot_layer: Dict[int, int] = {}       # cache slot -> index inside its group
        self.state: Dict[int, torch.Tensor] = {}   # cache slot -> [max_requests, *shape]
        self.n_slots = len(needs)
        by_key: Dict[tuple, CacheGroup] = {}
        for slot, need in enumerate(needs):
            items = need if isinstance(need, (list, tuple)) else [need]
            for item in items:
                if item is None:
                    continue
                if isinstance(item, PagedKVNeed):
                    if item.window is not None and item.window <= 0:
                        raise ValueError(f"cache slot {slot}: window {item.window} must be positive")
                    key = (item.n_kv_heads, item.head_dim, item.window)
                    g = by_key.get(key)
                    if g is None:
                        g = CacheGroup(len(self.groups), item, [], page_size, IdPool(num_pages, "page"))
                        by_key[key] = g
                        self.groups.append(g)
                    if slot in self.slot_group:
                        raise ValueError(f"cache slot {slot} asks for two paged caches")
                    self.slot_group[slot] = g.index
                    self.slot_layer[slot] = len(g.slots)
                    g.slots.append(slot)
                elif isinstance(item, StateNeed):
                    if allocate:
                        self.state[slot] = torch.zeros((max_requests,) + tuple(item.shape),
                                                       dtype=getattr(torch, item.dtype), device=self.device)
                    else:
                        self.state[slot] = None
                else:
                    raise TypeError(f"cache slot {slot}: unknown need {item!r}")
        if allocate:
            for g in self.groups:
                g.storage = torch.zeros((len(g.slots), 2, num_pages, g.need.n_kv_heads, page_size,
                                         g.need.head_dim), dtype=dtype, device=self.device)
        self.state_slots = IdPool(max_requests, "state slot")
        self.live: Dict[int, RequestCache] = {}
        self._next_rid = 0

    # ---- sizes -----------------------------------------------------------
    def bytes_per_page(self) -> int:
        """Device bytes that one more page in EVERY group's pool costs: keys and values of
        all layers of all groups (the pools have the same number of pages)."""
        esize = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.slots) * 2 * g.need.n_kv_heads * self.page_size * g.need.head_dim * esize
                   for g in self.groups)

    @classmethod
    def pages_within(cls, needs: Sequence, page_size: int, dtype: torch.dtype, budget_bytes: int) -> int:
        """How many pages per pool fit ``budget_bytes`` of device memory: the budget over
        ``bytes_per_page()`` (the reference's rule, pages = budget / (layers * 2 * page *
        kv width * element size); it sized a pool by a fixed count first and ran out of
        memory on a larger model, docs/JOURNAL.md:364-367, tools/modal_lab.py:232-240).
        Raises when not even one page fits."""
        per = cls(needs, page_size, 1, max_requests=1, dtype=dtype, allocate=False).bytes_per_page()
        if per == 0:
            return 1                  # no paged cache in this model: one page that nobody takes
        pages = int(budget_bytes) // per
        if pages < 1:
            raise ValueError(f"a cache budget of {int(budget_bytes)} bytes holds no page ({per} bytes each)")
        return pages

    def bytes_per_token_full(self) -> int:
        """Cache bytes that one more token of context costs in the groups that keep
        every key."""
        esize = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.slots) * 2 * g.need.n_kv_heads * g.need.head_dim * esize
                   for g in self.groups if g.window is None)

    def pages_ever_needed(self, total_tokens: int) -> List[int]:
        """Per group, the most pages a request of ``total_tokens`` tokens must hold at one
        time if it is fed in portions as small as need be.  A group that keeps every key
        needs a page for each ``page_size`` tokens; a window group only the pages that the
        window of one query can touch (the window's width, whatever its alignment, plus the
        page of the token being written), since the pages behind the window come back at
        every commit.  A model without any paged group needs none."""
        out = []
        for g in self.groups:
            pages = -(-int(total_tokens) // self.page_size)
            if g.window is not None:
                pages = min(pages, (g.window - 1) // self.page_size + 2)
            out.append(pages)
        return out

    def free_pages(self) -> List[int]:
        return [g.pool.free_count for g in self.groups]

    def used_pages(self) -> List[int]:
        return [g.pool.used_count for g in self.groups]

    # ---- requests --------------------------------------------------------
    def open(self, rid: Optional[int] = None) -> RequestCache:
        if rid is None:
            rid = self._next_rid
        self._next_rid = max(self._next_rid, rid + 1)
        if rid in self.live:
            raise CacheError(f"request {rid} is already open")
        (slot,) = self.state_slots.take(1)
        for t in self.state.values():
            if t is not None:
                t[slot].zero_()
        req = RequestCache(rid=rid, state_slot=slot, tables=[[] for _ in self.groups])
        self.live[rid] = req
        return req

    def _new_pages(self, req: RequestCache, n: int) -> List[int]:
        total = req.length + n
        need_pages = -(-total // self.page_size)
        return [max(0, need_pages - len(t)) for t in req.tables]

    def can_reserve(self, req: RequestCache, n: int) -> bool:
        return all(c <= g.pool.free_count for c, g in zip(self._new_pages(req, n), self.groups))

    def can_reserve_all(self, wants: Sequence) -> bool:
        """True if every (request, n) of ``wants`` can be reserved together."""
        totals = [0] * len(self.groups)
        for req, n in wants:
            for i, c in enumerate(self._new_pages(req, n)):
                totals[i] += c
        return all(t <= g.pool.free_count for t, g in zip(totals, self.groups))

    def room_for(self, req: RequestCache, planned_pages: Optional[Sequence[int]] = None) -> int:
        """How many more tokens ``req`` could reserve now, if ``planned_pages[g]`` pages
        of each group are already promised to others."""
        room = None
        for i, (g, table) in enumerate(zip(self.groups, req.tables)):
            free = g.pool.free_count - (planned_pages[i] if planned_pages else 0)
            r = (len(table) + max(0, free)) * self.page_size - req.length
            room = r if room is None else min(room, r)
        return max(0, room) if room is not None else (1 << 30)

    def pages_for(self, req: RequestCache, n: int) -> List[int]:
        """New pages per group that reserving ``n`` more tokens would take."""
        return self._new_pages(req, n)

    def reserve(self, req: RequestCache, n: int) -> None:
        """Make the tables cover ``n`` more tokens than are committed.  Raises
        ``OutOfPages`` with nothing taken when any group cannot provide."""
        self._check_open(req)
        if n < 0:
            raise ValueError("cannot reserve a negative number of tokens")
        counts = self._new_pages(req, n)
        for c, g in zip(counts, self.groups):
            if c > g.pool.free_count:
                raise OutOfPages(f"request {req.rid}: group {g.index} needs {c} more pages, "
                                 f"{g.pool.free_count} of {g.pool.n} free")
        for c, g, table in zip(counts, self.groups, req.tables):
            table.extend(g.pool.take(c))

    def commit(self, req: RequestCache, n: int) -> None:
        """``n`` tokens were written.  Window groups give back the pages that no
        later query can see."""
        self._check_open(req)
        total = req.length + n
        for table in req.tables:
            if total > len(table) * self.page_size:
                raise CacheError(f"request {req.rid}: commit of {n} tokens beyond its reservation")
        req.length = total
        for g, table in zip(self.groups, req.tables):
            if g.window is None:
                continue
            first_needed = total + 1 - g.window      # earliest key the next query reads
            dead = max(0, first_needed) // self.page_size
            for j in range(min(dead, len(table))):
                if table[j] >= 0:
                    g.pool.give([table[j]])
                    table[j] = -1

    def trim_reservation(self, req: RequestCache) -> None:
        """Give back pages reserved beyond the committed length (a step that did not run)."""
        self._check_open(req)
        keep = -(-req.length // self.page_size)
        for g, table in zip(self.groups, req.tables):
            extra = [p for p in table[keep:] if p >= 0]
            g.pool.give(extra)
            del table[keep:]

    def close(self, req: RequestCache) -> None:
        self._check_open(req)
        for g, table in zip(self.groups, req.tables):
            g.pool.give([p for p in table if p >= 0])
            table.clear()
        self.state_slots.give([req.state_slot])
        req.closed = True
        req.length = 0
        del self.live[req.rid]

    def _check_open(self, req: RequestCache) -> None:
        if req.closed or self.live.get(req.rid) is not req:
            raise CacheError(f"request {req.rid} is not open in this cache")

    # ---- views for the model ---------------------------------------------
    def layer_caches(self, block_tables: Dict[int, torch.Tensor]) -> List[LayerCache]:
        """One ``LayerCache`` per cache slot, with this step's device block tables."""
        out = []
        for slot in range(self.n_slots):
            k = v = table = None
            if slot in self.slot_group:
                g = self.groups[self.slot_group[slot]]
                layer = self.slot_layer[slot]
                k, v = g.storage[layer, 0], g.storage[layer, 1]
                table = block_tables[g.index]
            out.append(LayerCache(k=k, v=v, block_table=table, state=self.state.get(slot),
                                  writes=True, page_size=self.page_size))
        return out

    # ---- checks for tests and debugging -------------------------------------
    def audit(self) -> None:
        """Every page is either free or held by exactly one live request."""
        for g in self.groups:
            held = [p for r in self.live.values() for p in r.tables[g.index] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g.index}: a page is held twice")
            if len(held) + g.pool.free_count != g.pool.n:
                raise CacheError(f"group {g.index}: {g.pool.n - len(held) - g.pool.free_count} pages lost")
            if set(held) & set(g.pool._free):
                raise CacheError(f"group {g.index}: a held page is on the free list")
        slots = [r.state_slot for r in self.live.values()]
        if len(slots) != len(set(slots)) or len(slots) + self.state_slots.free_count != self.state_slots.n:
            raise CacheError("state slots are lost or held twice")
