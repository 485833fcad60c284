"""The cache manager: what every live request holds, on the host.

Two kinds of holdings, both decided by what the model's mixers ask for:

* **paged groups** - mixers whose cache grows with the sequence (keys and values). Mixers
  with the same need (element type, heads, head size, window) form a group; a group has its
  own page pool and each request one block table per group. One page id covers
  ``page_tokens`` positions of every layer of the group, as celeg's page layout does
  (include/celeg/runtime/cache/page_layout.hpp:89-98). A group with a window gives a page
  back as soon as every position in it is older than the window of the next query.
* **state slots** - mixers with per-request state of fixed size. One slot holds the state of
  all such layers of one request; a slot is cleared when a request takes it (celeg zeroes the
  conv state at reset: src/backend/cpu/model_state.cpp:395-397).

Everything a request holds is given back in one place, :meth:`CacheManager.close`, as celeg
does in ``finish_request_locked`` (src/backend/cuda/runtime/request_lifecycle.cpp:200-218).
This module holds no device memory; :mod:`celeg_b200.cache.storage` does.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from .pages import OutOfPages, PageError, PagePool

NO_PAGE = -1


@dataclass(frozen=True)
class PagedNeed:
    """A cache that grows per position by ``kv_heads * head_dim`` elements for keys and by
    ``kv_heads * value_head_dim`` for values (``None``: as wide as the keys; 0: nothing is kept beside the
    keys, as for a mixer that caches one latent vector per position); ``window`` = how many most recent
    positions (the query's own included) a query may read, ``None`` = all."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_head_dim: Optional[int] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.value_head_dim is None else self.value_head_dim

    def group_key(self) -> tuple:
        return ("paged", self.kv_heads, self.head_dim, self.window, self.value_dim)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: ``elements`` 32-bit floats, zero for a new request."""
    elements: int


@dataclass
class PagedGroup:
    key: tuple
    need: PagedNeed
    pool: PagePool
    members: List[Hashable] = field(default_factory=list)  # places (run-order position, part name) that own a layer of this group

    @property
    def window(self) -> Optional[int]:
        return self.need.window


@dataclass
class StateLayout:
    # keyed by the place of the state in the model: (position of the run order, name of the part)
    offsets: Dict[Hashable, int] = field(default_factory=dict)  # place -> first float in the slot
    sizes: Dict[Hashable, int] = field(default_factory=dict)
    slot_elements: int = 0

    def add(self, position: Hashable, elements: int) -> int:
        offset = self.slot_elements
        self.offsets[position] = offset
        self.sizes[position] = elements
        # keep every layer's state 16-byte aligned for vector loads
        self.slot_elements += (elements + 3) // 4 * 4
        return offset


@dataclass
class RequestCache:
    """What one live request holds."""
    request_id: Hashable
    slot: int
    tokens: int = 0                                          # positions already written
    tables: List[List[int]] = field(default_factory=list)    # per group: logical page index -> page id / NO_PAGE
    first_live_page: List[int] = field(default_factory=list)  # per group: pages below it were given back
    closed: bool = False
    # per group: the same table as an int32 array (capacity >= length), kept in step with ``tables`` by the
    # manager, so that a step copies a request's table into its staging buffer with one memcpy; with a
    # manager that keeps table mirrors these are rows of the mirrors (one row per slot)
    arrays: List[np.ndarray] = field(default_factory=list)
    # positions that fit into the pages held (the smallest group decides): while a request stays below it,
    # no page has to be found for it and nobody needs to look at its tables
    capacity: int = 0
    page_tokens: int = 0

    def held_pages(self, group: int) -> List[int]:
        return [page for page in self.tables[group] if page != NO_PAGE]

    def table_array(self, group: int) -> np.ndarray:
        """The block table of ``group`` as int32, one entry per logical page."""
        return self.arrays[group][:len(self.tables[group])]

    def _append(self, group: int, pages: Sequence[int]) -> None:
        table = self.tables[group]
        start = len(table)
        table.extend(pages)
        array = self.arrays[group]
        if len(table) > array.shape[0]:
            # (a row of a mirror is as long as the longest context needs; a table that outgrows it is a
            # request past the context limit, which the step function refuses: the row is left behind)
            grown = np.full(max(len(table), 2 * array.shape[0], 16), NO_PAGE, dtype=np.int32)
            grown[:start] = array[:start]
            self.arrays[group] = array = grown
        array[start:len(table)] = pages
        self.capacity = min(len(t) for t in self.tables) * self.page_tokens


class CacheManager:
    def __init__(self, page_tokens: int, group_pages: Sequence[int], groups: Sequence[Tuple[tuple, PagedNeed]],
                 state_layout: StateLayout, slots: int,
                 clear_slot: Optional[Callable[[int], None]] = None, table_capacity: Optional[int] = None):
        """``table_capacity``: with a number, the manager keeps every group's block tables of all slots in one
        int32 array ``table_mirrors[group][slot, :table_capacity]`` (NO_PAGE where a request holds nothing), so
        that a step gathers the tables of its requests with one indexing operation."""
        if len(group_pages) != len(groups):
            raise ValueError("one page count per paged group is needed")
        self.page_tokens = page_tokens
        self.table_mirrors: Optional[List[np.ndarray]] = None
        if table_capacity is not None:
            self.table_mirrors = [np.full((slots, max(1, table_capacity)), NO_PAGE, dtype=np.int32) for _ in groups]
        self.groups: List[PagedGroup] = [
            PagedGroup(key=key, need=need, pool=PagePool(pages, page_tokens))
            for (key, need), pages in zip(groups, group_pages)]
        self.state_layout = state_layout
        self._free_slots: List[int] = list(range(slots - 1, -1, -1))
        self.total_slots = slots
        self._clear_slot = clear_slot
        self._live: Dict[Hashable, RequestCache] = {}
        self._any_window = any(group.window is not None for group in self.groups)

    # ------------------------------------------------------------------ queries
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def live_requests(self) -> List[Hashable]:
        return list(self._live)

    def get(self, request_id: Hashable) -> RequestCache:
        try:
            return self._live[request_id]
        except KeyError:
            raise KeyError(f"request {request_id!r} holds no cache") from None

    def find(self, request_id: Hashable) -> Optional[RequestCache]:
        """The request's holdings, or None if it holds nothing."""
        return self._live.get(request_id)

    def pages_needed(self, cache: RequestCache, new_total: int) -> List[int]:
        """Per group, how many pages must be added for positions ``[cache.tokens, new_total)``."""
        out = []
        for index, group in enumerate(self.groups):
            have = len(cache.tables[index])
            out.append(max(0, group.pool.pages_for(new_total) - have))
        return out

    def pages_needed_each(self, caches: Sequence[RequestCache], counts: Sequence[int]) -> List[int]:
        """Per group, the pages that must be added so that every ``caches[i]`` can take ``counts[i]`` more
        positions. A request that stays within the pages it holds is passed over without a look at its tables."""
        total = [0] * len(self.groups)
        for cache, count in zip(caches, counts):
            if cache.tokens + count > cache.capacity:
                for index, pages in enumerate(self.pages_needed(cache, cache.tokens + count)):
                    total[index] += pages
        return total

    def reserve_each(self, caches: Sequence[RequestCache], counts: Sequence[int]) -> None:
        """:meth:`reserve` for every ``caches[i]`` up to ``counts[i]`` more positions (the caller has checked
        with :meth:`pages_needed_each` that the pools hold enough)."""
        for cache, count in zip(caches, counts):
            if cache.tokens + count > cache.capacity:
                self.reserve(cache, cache.tokens + count)
            elif cache.closed:
                raise PageError(f"request {cache.request_id!r} was closed")

    def advance_each(self, caches: Sequence[RequestCache], counts: Sequence[int]) -> None:
        """:meth:`advance` for every ``caches[i]`` by ``counts[i]`` positions."""
        if self._any_window:
            for cache, count in zip(caches, counts):
                self.advance(cache, cache.tokens + count)
            return
        for cache, count in zip(caches, counts):
            if count < 0:
                raise ValueError("a request's length cannot shrink")
            if cache.tokens + count > cache.capacity:
                raise PageError(f"request {cache.request_id!r} advanced to {cache.tokens + count} positions "
                                f"without pages")
            cache.tokens += count

    def can_hold(self, tokens: int) -> bool:
        """Whether a NEW request of ``tokens`` positions could be given its slot and pages now."""
        if not self._free_slots:
            return False
        return all(group.pool.free_pages >= self._steady_pages(group, tokens) for group in self.groups)

    def _steady_pages(self, group: PagedGroup, tokens: int) -> int:
        pages = group.pool.pages_for(tokens)
        if group.window is not None:
            # a window of w positions touches at most ceil((w-1)/P)+1 pages, plus the pages of
            # the portion being written before old ones are given back
            pages = min(pages, group.pool.pages_for(group.window - 1) + 1 + 1)
        return pages

    # ---------------------------------------------------------------- lifecycle
    def open(self, request_id: Hashable) -> RequestCache:
        """Take a slot (cleared) for a new request; it holds no pages yet."""
        if request_id in self._live:
            raise ValueError(f"request {request_id!r} already holds a cache")
        if not self._free_slots:
            raise OutOfPages("no state slot is free")
        slot = self._free_slots.pop()
        if self._clear_slot is not None:
            self._clear_slot(slot)
        if self.table_mirrors is not None:
            arrays = [mirror[slot] for mirror in self.table_mirrors]           # (NO_PAGE throughout: see close)
        else:
            arrays = [np.full(16, NO_PAGE, dtype=np.int32) for _ in self.groups]
        cache = RequestCache(request_id=request_id, slot=slot,
                             tables=[[] for _ in self.groups],
                             first_live_page=[0 for _ in self.groups],
                             arrays=arrays, page_tokens=self.page_tokens)
        self._live[request_id] = cache
        return cache

    def reserve(self, cache: RequestCache, new_total: int) -> None:
        """Make room for positions up to ``new_total`` in every group, all or nothing."""
        if cache.closed:
            raise PageError(f"request {cache.request_id!r} was closed")
        needed = self.pages_needed(cache, new_total)
        for group, count in zip(self.groups, needed):
            if group.pool.free_pages < count:
                raise OutOfPages(
                    f"request {cache.request_id!r} needs {count} more page(s) of group {group.key}, "
                    f"{group.pool.free_pages} free")
        for index, (group, count) in enumerate(zip(self.groups, needed)):
            taken = group.pool.allocate(count)
            assert taken is not None
            if taken:
                cache._append(index, taken)

    def advance(self, cache: RequestCache, new_total: int) -> List[Tuple[int, int]]:
        """Record that positions below ``new_total`` are written; give back pages that no later
        query can read. Returns the (group, page) pairs that were released."""
        if new_total < cache.tokens:
            raise ValueError("a request's length cannot shrink")
        for index, group in enumerate(self.groups):
            if group.pool.pages_for(new_total) > len(cache.tables[index]):
                raise PageError(f"request {cache.request_id!r} advanced to {new_total} positions without pages")
        cache.tokens = new_total
        released: List[Tuple[int, int]] = []
        for index, group in enumerate(self.groups):
            if group.window is None:
                continue
            # the next query sits at position new_total and reads positions > new_total - window
            first_needed = max(0, new_total - group.window + 1)
            first_page = first_needed // self.page_tokens
            table = cache.tables[index]
            for logical in range(cache.first_live_page[index], min(first_page, len(table))):
                page = table[logical]
                if page != NO_PAGE:
                    group.pool.release([page])
                    table[logical] = NO_PAGE
                    cache.arrays[index][logical] = NO_PAGE
                    released.append((index, page))
            cache.first_live_page[index] = max(cache.first_live_page[index], min(first_page, len(table)))
        return released

    def close(self, request_id: Hashable) -> None:
        """Give back everything the request holds. Closing twice is an error."""
        cache = self._live.pop(request_id, None)
        if cache is None:
            raise PageError(f"request {request_id!r} holds no cache (closed twice?)")
        for index, group in enumerate(self.groups):
            group.pool.release(cache.held_pages(index))
            used = len(cache.tables[index])
            cache.tables[index] = []
            if self.table_mirrors is not None:
                self.table_mirrors[index][cache.slot, :used] = NO_PAGE
        cache.capacity = 0
        self._free_slots.append(cache.slot)
        cache.closed = True

    # ----------------------------------------------------------------- checking
    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held; the same for slots."""
        for index, group in enumerate(self.groups):
            held: Dict[int, Hashable] = {}
            for cache in self._live.values():
                for page in cache.held_pages(index):
                    if page in held:
                        raise PageError(f"page {page} of group {group.key} is held by {held[page]!r} "
                                        f"and {cache.request_id!r}")
                    held[page] = cache.request_id
                    if group.pool.ref_count(page) != 1:
                        raise PageError(f"page {page} of group {group.key} is held with ref count "
                                        f"{group.pool.ref_count(page)}")
            if len(held) != group.pool.used_pages:
                raise PageError(f"group {group.key}: {group.pool.used_pages} pages are out of the pool, "
                                f"requests hold {len(held)}")
        slots = [cache.slot for cache in self._live.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise PageError("a state slot is held twice or is both free and held")
        if len(slots) + len(self._free_slots) != self.total_slots:
            raise PageError("a state slot was lost")
