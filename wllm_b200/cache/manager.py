"""The cache manager: pages of keys and values per group of layers, a block table per
request and group, and slots for per-request state of fixed size.

A *group* is a set of layers with the same needs: number of key/value heads, head
size and how much of the past they read (all of it, or a window).  Every group has
its own pool of pages and its own table per request; one page of a group holds
`page_size` tokens of all the group's layers.  Pages are taken when a step reserves
room for new tokens and given back when the request is closed, or, in a window
group, as soon as no later token can read them.  Reserving for a step is atomic:
either every request of the step gets its pages or nothing changes and
`OutOfPages` is raised, which is how the scheduler learns that it has to preempt.

Beside the pages, every live request owns one *slot*: a row index into the state
tensors (per-request state of fixed size that a mixer may declare, for instance a
recurrent state) and, for the engine, a stable small integer for the request.
Gemma 1 declares no state; the slot is still taken and given back.

Reference for the bookkeeping this replaces: src/wllm/engine/kv_cache.py:63-303
(one table per sequence shared by all layers, reserve/advance, free_sequence).
Pool layout on the device, per group:
    [layer_in_group][k|v][page][kv_head][slot_in_page][head_dim]
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .pages import OutOfPages, PagePool


@dataclass(frozen=True)
class CacheGroupSpec:
    name: str
    layers: int            # cache layers in the group
    kv_heads: int
    head_dim: int
    window: int | None = None   # None: every key is kept; n: a token reads the n latest keys (itself included)


@dataclass(frozen=True)
class StateSpec:
    name: str
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class RequestCache:
    """What one live request holds.  `tables[g][i]` is the page with tokens
    i*page_size .. (i+1)*page_size-1 in group g, or -1 once a window has passed it."""
    request_id: object
    slot: int
    tables: list
    num_tokens: int = 0        # tokens whose keys and values are written and committed
    reserved: int = 0          # tokens reserved by the step in flight
    closed: bool = False
    released_upto: list = field(default_factory=list)   # per group: pages below this index were given back
    version: int = 0           # bumped whenever a table changes (lets a reader cache a copy)


class CacheGroup:
    def __init__(self, spec: CacheGroupSpec, num_pages: int, page_size: int, dtype, device, poison: bool = False):
        self.spec = spec
        self.pool = PagePool(num_pages)
        self.page_size = page_size
        self.pages = None
        self.poison = poison
        if device is not None:
            shape = (spec.layers, 2, num_pages, spec.kv_heads, page_size, spec.head_dim)
            self.pages = torch.full(shape, float("nan"), dtype=dtype, device=device) if poison else \
                torch.zeros(shape, dtype=dtype, device=device)

    def give(self, pages: list) -> None:
        """Pages go back to the pool; with `poison` their contents become NaN first (in stream order, so a step
        still running has read them before)."""
        if self.poison and self.pages is not None and pages:
            index = torch.tensor(pages, dtype=torch.long, device=self.pages.device)
            self.pages.index_fill_(2, index, float("nan"))
        for page in pages:
            self.pool.give(page)

    def keys(self, layer: int) -> torch.Tensor:
        return self.pages[layer, 0]

    def values(self, layer: int) -> torch.Tensor:
        return self.pages[layer, 1]

    def bytes_per_token(self) -> int:
        item = 4 if self.pages is None else self.pages.element_size()
        return self.spec.layers * 2 * self.spec.kv_heads * self.spec.head_dim * item


class StateSlots:
    """Rows of fixed-size per-request state: tensor `name` has shape [num_slots, *shape]."""

    def __init__(self, num_slots: int, specs: list, device):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots
        self.tensors = {}
        if device is not None:
            for s in specs:
                self.tensors[s.name] = torch.zeros((num_slots,) + tuple(s.shape), dtype=s.dtype, device=device)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("request slots", 1, 0)
        slot = self._free.pop()
        self._held[slot] = True
        for t in self.tensors.values():   # a new request starts from zero state
            t[slot].zero_()
        return slot

    def give(self, slot: int) -> None:
        if not self._held[slot]:
            raise RuntimeError(f"state slot {slot} given back but not held")
        self._held[slot] = False
        self._free.append(slot)


class CacheManager:
    def __init__(self, groups: list, page_size: int, num_pages: int, max_requests: int, states: list = (),
                 dtype=torch.bfloat16, device=None, poison: bool = False):
        """`poison` (a debugging aid; the tests switch it on): pools start as NaN instead of zeros and every
        page is filled with NaN again when it is given back, so a kernel that reads a slot that was never
        written, or a page that its request no longer holds, shows at once in the logits."""
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.groups = [CacheGroup(g, num_pages, page_size, dtype, device, poison) for g in groups]
        self.slots = StateSlots(max_requests, list(states), device)
        self.live: dict = {}
        self.dtype, self.device = dtype, device
        self.pages_high_water = [0] * len(self.groups)

    # -- requests ------------------------------------------------------------------
    def open(self, request_id) -> RequestCache:
        if request_id in self.live:
            raise KeyError(f"request {request_id!r} is already open")
        rc = RequestCache(request_id, self.slots.take(), [[] for _ in self.groups],
                          released_upto=[0] * len(self.groups))
        self.live[request_id] = rc
        return rc

    def close(self, rc: RequestCache) -> None:
        """Give back everything the request holds.  Closing twice is an error."""
        if rc.closed:
            raise RuntimeError(f"request {rc.request_id!r} closed twice")
        for g, table in zip(self.groups, rc.tables):
            g.give([page for page in reversed(table) if page >= 0])
            table.clear()
        self.slots.give(rc.slot)
        rc.closed = True
        del self.live[rc.request_id]

    # -- pages ---------------------------------------------------------------------
    def _pages_for(self, rc: RequestCache, extra: int) -> int:
        total = rc.num_tokens + rc.reserved + extra
        return -(-total // self.page_size)

    def pages_needed(self, wants: list) -> list:
        """Pages that each group must hand out so that every (request, n_new) of `wants` fits."""
        need = [0] * len(self.groups)
        for rc, n in wants:
            target = self._pages_for(rc, n)
            for gi in range(len(self.groups)):
                need[gi] += max(0, target - len(rc.tables[gi]))
        return need

    def can_reserve(self, wants: list) -> bool:
        return all(n <= g.pool.num_free for n, g in zip(self.pages_needed(wants), self.groups))

    def reserve(self, wants: list) -> None:
        """Take the pages for all of `wants` = [(request, n_new_tokens)], or none of them."""
        need = self.pages_needed(wants)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(g.spec.name, n, g.pool.num_free)
        for rc, n in wants:
            if rc.closed:
                raise RuntimeError(f"request {rc.request_id!r} is closed")
            target = self._pages_for(rc, n)
            for g, table in zip(self.groups, rc.tables):
                while len(table) < target:
                    table.append(g.pool.take())
                    rc.version += 1
            rc.reserved += n
        for gi, g in enumerate(self.groups):
            used = g.pool.num_pages - g.pool.num_free
            self.pages_high_water[gi] = max(self.pages_high_water[gi], used)

    def token_slots(self, rc: RequestCache, group: int, start: int, n: int) -> list:
        """Flat slots (page * page_size + offset) of the tokens start .. start+n-1 of a request."""
        table, ps = rc.tables[group], self.page_size
        return [table[p // ps] * ps + p % ps for p in range(start, start + n)]

    def commit(self, rc: RequestCache, n: int) -> None:
        """The step wrote `n` reserved tokens.  Window groups give back the pages that
        no later token can read: a token at position p reads keys p-window+1 .. p."""
        if n > rc.reserved:
            raise RuntimeError("commit of more tokens than reserved")
        rc.reserved -= n
        rc.num_tokens += n
        for gi, g in enumerate(self.groups):
            w = g.spec.window
            if w is None:
                continue
            first_needed = rc.num_tokens - w + 1          # oldest key the next token reads
            upto = min(max(0, first_needed // self.page_size), len(rc.tables[gi]))
            passed = list(range(rc.released_upto[gi], upto))
            g.give([rc.tables[gi][i] for i in passed])
            for i in passed:
                rc.tables[gi][i] = -1
                rc.version += 1
            rc.released_upto[gi] = max(rc.released_upto[gi], upto)

    def cancel_reservation(self, rc: RequestCache) -> None:
        """Undo a reservation that no step used: surplus pages go back."""
        rc.reserved = 0
        target = -(-rc.num_tokens // self.page_size)
        for g, table in zip(self.groups, rc.tables):
            surplus = []
            while len(table) > target:
                page = table.pop()
                rc.version += 1
                if page >= 0:          # (a window never passes a page that holds no committed token; checked all the same)
                    surplus.append(page)
            g.give(surplus)

    # -- figures -------------------------------------------------------------------
    def free_pages(self) -> list:
        return [g.pool.num_free for g in self.groups]

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)

    def check(self) -> None:
        """Every page is either free or in exactly one live table; used by the tests."""
        for gi, g in enumerate(self.groups):
            seen = {}
            for rc in self.live.values():
                for page in rc.tables[gi]:
                    if page < 0:
                        continue
                    if page in seen:
                        raise AssertionError(f"group {g.spec.name}: page {page} held by {seen[page]!r} and {rc.request_id!r}")
                    if not g.pool.is_held(page):
                        raise AssertionError(f"group {g.spec.name}: page {page} is in a table but free")
                    seen[page] = rc.request_id
            if len(seen) + g.pool.num_free != g.pool.num_pages:
                raise AssertionError(f"group {g.spec.name}: {g.pool.num_pages - g.pool.num_free - len(seen)} pages lost")
