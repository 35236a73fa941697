"""Cache manager: page ids, block tables and state slots.  Owns no device memory.

Pages.  Keys and values live in pages of `page_size` tokens.  Caches with the same
needs (kv heads, head size, window) form a group; every group has a pool of pages
of its own and every request one block table per group.  Logical block i of a
request covers positions [i * page_size, (i + 1) * page_size).

What follows Azimml/shrike's BlockManager (shrike/engine/block_manager.py): a FIFO
free list handed out from the left and refilled on the right (:38,51-58,121-126),
reference counts (:21-27), demand = ceil((computed + new) / page_size) - held
(:60-70), `can_append` = demand <= free (:72-73), allocation of exactly the demand
(:75-77), everything returned on free (:128-130).  Prefix caching is left out.

Beyond it: groups, each with a pool sized for its own need (a group whose layers see a
window of keys holds far fewer pages per request than one that keeps them all); giving pages
back while a request lives, once a window has passed them (their table entry becomes -1); and
slots for per-request state of fixed size, taken with the first pages and returned with the
last.  Slots handed out since the last step are remembered (`take_opened`), so that the step
function can zero their state before a new request's first token runs.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np


class CacheError(RuntimeError):
    """Bookkeeping was asked to do something impossible (double free, no page)."""


@dataclass(frozen=True)
class KVGroupSpec:
    cache_ids: tuple[int, ...]
    num_kv_heads: int
    head_dim: int
    window: int | None = None


class IdPool:
    """A fixed set of ids with reference counts and a FIFO free list."""

    def __init__(self, count: int):
        self.count = count
        self.free_queue: deque[int] = deque(range(count))
        self.ref_count = [0] * count

    @property
    def num_free(self) -> int:
        return len(self.free_queue)

    def take(self) -> int:
        if not self.free_queue:
            raise CacheError("no free id left")
        ident = self.free_queue.popleft()
        if self.ref_count[ident] != 0:
            raise CacheError(f"id {ident} was on the free list while held")
        self.ref_count[ident] = 1
        return ident

    def share(self, ident: int) -> None:
        if self.ref_count[ident] < 1:
            raise CacheError(f"id {ident} is not held, cannot be shared")
        self.ref_count[ident] += 1

    def give_back(self, ident: int) -> None:
        if not 0 <= ident < self.count or self.ref_count[ident] < 1:
            raise CacheError(f"id {ident} given back but not held")
        self.ref_count[ident] -= 1
        if self.ref_count[ident] == 0:
            self.free_queue.append(ident)


class BlockTable:
    """One request's pages in one group: a growing int32 array, -1 where a page
    has been given back."""

    __slots__ = ("pages", "length", "released")

    def __init__(self):
        self.pages = np.full(8, -1, dtype=np.int32)
        self.length = 0
        self.released = 0  # leading entries already given back

    def append(self, page: int) -> None:
        if self.length == len(self.pages):
            grown = np.full(2 * len(self.pages), -1, dtype=np.int32)
            grown[: self.length] = self.pages[: self.length]
            self.pages = grown
        self.pages[self.length] = page
        self.length += 1

    def view(self) -> np.ndarray:
        return self.pages[: self.length]

    def tolist(self) -> list[int]:
        return self.view().tolist()


@dataclass
class RequestCache:
    """What one live request holds."""

    tables: list[BlockTable]
    slot: int = -1
    live: bool = field(default=True)


class CacheManager:
    def __init__(self, groups: list[KVGroupSpec], page_size: int, num_pages, max_slots: int):
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        self.groups = list(groups)
        self.page_size = page_size
        counts = [num_pages] * len(self.groups) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(self.groups):
            raise ValueError("one page count per group")
        self.pools = [IdPool(count) for count in counts]
        self.slots = IdPool(max_slots)
        self.has_windows = any(group.window is not None for group in self.groups)
        self._opened: list[int] = []   # slots handed out since `take_opened` was last called

    # ---- figures -----------------------------------------------------------
    @property
    def num_pages(self) -> list[int]:
        return [pool.count for pool in self.pools]

    @property
    def num_free(self) -> list[int]:
        return [pool.num_free for pool in self.pools]

    @property
    def main_pool(self) -> IdPool | None:
        """The largest pool: the one a user's "number of KV blocks" speaks of (None without pages)."""
        return max(self.pools, key=lambda pool: pool.count) if self.pools else None

    @property
    def total_pages(self) -> int:
        return self.main_pool.count if self.pools else 0

    @property
    def free_pages(self) -> int:
        return self.main_pool.num_free if self.pools else 0

    def portion_limit(self) -> int | None:
        """The longest portion one request can be fed in a step, whatever else is free: a group
        with a window must hold the window and the portion at once (None: no such bound)."""
        limits = [max(1, (pool.count - 2) * self.page_size - group.window + 2)
                  for pool, group in zip(self.pools, self.groups) if group.window is not None]
        return min(limits) if limits else None

    def whole(self) -> bool:
        """True when nothing is held: every page and every slot is free."""
        return all(p.num_free == p.count for p in self.pools) and self.slots.num_free == self.slots.count

    def blocks_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def worst_case_pages(self, tokens: int, portion: int | None = None) -> list[int]:
        """Pages per group a request of `tokens` may hold at once when it is fed at most `portion`
        tokens a step (None: all at once).  A group with a window holds the pages that the
        window and the portion in flight touch, whatever the request's length."""
        return [pages_in_flight(self.blocks_for(tokens), group.window, min(portion or tokens, tokens), self.page_size)
                for group in self.groups]

    # ---- a request's life ----------------------------------------------------
    def open(self) -> RequestCache:
        """Takes a state slot; pages come with `append`."""
        slot = self.slots.take()
        self._opened.append(slot)
        return RequestCache(tables=[BlockTable() for _ in self.groups], slot=slot)

    def take_opened(self) -> list[int]:
        """The state slots handed out since the last call: what the step function zeroes."""
        opened, self._opened = self._opened, []
        return opened

    def can_open(self) -> bool:
        return self.slots.num_free > 0

    def pages_needed(self, cache: RequestCache, num_computed: int, num_new: int) -> list[int]:
        total = self.blocks_for(num_computed + num_new)
        return [max(0, total - table.length) for table in cache.tables]

    def can_append(self, cache: RequestCache | None, num_computed: int, num_new: int) -> bool:
        if cache is None:  # not opened yet: needs a slot too
            total = self.blocks_for(num_computed + num_new)
            return self.can_open() and all(total <= pool.num_free for pool in self.pools)
        needed = self.pages_needed(cache, num_computed, num_new)
        return all(n <= pool.num_free for n, pool in zip(needed, self.pools))

    def append(self, cache: RequestCache, num_computed: int, num_new: int) -> None:
        if not cache.live:
            raise CacheError("append on a request whose cache was freed")
        needed = self.pages_needed(cache, num_computed, num_new)
        if any(n > pool.num_free for n, pool in zip(needed, self.pools)):
            raise CacheError("append without room; call can_append first")
        for table, pool, count in zip(cache.tables, self.pools, needed):
            for _ in range(count):
                table.append(pool.take())

    def has_room(self, cache: RequestCache, total_tokens: int) -> bool:
        """True when the pages already held cover `total_tokens` in every group (nothing to take)."""
        limit = total_tokens
        size = self.page_size
        for table in cache.tables:
            if table.length * size < limit:
                return False
        return True

    def advance(self, cache: RequestCache, num_computed: int) -> int:
        """After a step: gives back the pages that every later query's window has
        passed.  The next query sits at position `num_computed` and sees keys from
        `num_computed - window + 1` on.  Returns how many pages were given back."""
        if not self.has_windows:
            return 0
        given = 0
        for table, pool, group in zip(cache.tables, self.pools, self.groups):
            if group.window is None:
                continue
            first_needed = num_computed - group.window + 1
            passed = min(max(0, first_needed // self.page_size), table.length)
            for index in range(table.released, passed):
                pool.give_back(int(table.pages[index]))
                table.pages[index] = -1
                given += 1
            table.released = max(table.released, passed)
        return given

    def free(self, cache: RequestCache) -> None:
        """Gives back everything the request holds; a second call is an error."""
        if not cache.live:
            raise CacheError("request cache freed twice")
        for table, pool in zip(cache.tables, self.pools):
            for page in table.view():
                if page >= 0:
                    pool.give_back(int(page))
            table.length = 0
            table.released = 0
        self.slots.give_back(cache.slot)
        cache.slot = -1
        cache.live = False


def pages_in_flight(whole: int, window: int | None, portion: int, page_size: int) -> int:
    """Pages one request holds at most in a group: all `whole` of them, or, with a window, those
    from the first key the portion's first query still sees to the portion's last token."""
    if window is None:
        return whole
    return min(whole, (window + portion - 2) // page_size + 2)


def pages_per_group(groups, page_size: int, budget_bytes: int, bytes_per_page: list[int], max_slots: int,
                    max_portion: int) -> list[int]:
    """Page counts for a budget of bytes: every group without a window gets the same count N, a
    group with a window at most what `max_slots` requests fed `max_portion` tokens a step can
    hold of it; N is as large as the budget allows."""
    caps = [None if group.window is None else max_slots * pages_in_flight(1 << 40, group.window, max_portion, page_size)
            for group in groups]
    capped: set[int] = set()
    while True:
        spent = sum(caps[g] * bytes_per_page[g] for g in capped)
        rest = sum(bytes_per_page[g] for g in range(len(groups)) if g not in capped)
        if rest == 0:
            return [caps[g] for g in range(len(groups))]
        count = max(0, budget_bytes - spent) // rest
        over = {g for g in range(len(groups)) if g not in capped and caps[g] is not None and caps[g] < count}
        if not over:
            return [caps[g] if g in capped else count for g in range(len(groups))]
        capped |= over


def group_caches(needs: dict[int, object]) -> list[KVGroupSpec]:
    """Groups cache ids whose KVNeed is identical; order of first appearance."""
    groups: dict[tuple, list[int]] = {}
    for cache_id in sorted(needs):
        need = needs[cache_id]
        key = (need.num_kv_heads, need.head_dim, need.window)
        groups.setdefault(key, []).append(cache_id)
    return [KVGroupSpec(tuple(ids), *key) for key, ids in groups.items()]
