"""Host side of the cache: pages, block tables, groups of layers, and slots for fixed-size state.

Parity with the reference's ``BlockAllocator`` and ``PagedKVCache``
(src/cloud_engine/cache.py:80-155, 235-529): a LIFO free list with an owner map, so a page
has zero or one owner and a double or foreign free is an error that changes nothing
(cache.py:132-145); requests are admitted with an empty table (engine.py:218-219); several
tables grow in one all-or-nothing transaction before a step (cache.py:371-396); lengths are
committed only after the step ran (cache.py:427-431); a request's pages all come back when
it ends or is preempted (cache.py:497-501).

Beyond the reference (which has one group and no state):

* **Groups.** Layers whose mixers need the same thing of the cache (all keys, or a window
  of them; same heads and head size) form a group with a page pool, an allocator and block
  tables of its own.  A page id is valid for every layer of its group.
* **Windows.** In a group with ``window`` W > 0 a query at position p reads keys
  p-W+1..p only, so once a request's committed length is n every page that lies wholly
  below n-W+1 is given back at once and its table entry becomes -1.
* **State slots.** Every admitted request holds one slot id; mixers with per-request
  state of fixed size index their state tensors with it.  A slot is marked dirty at
  admission so that the device side zeroes the state before the request's first step.

This module touches no device and imports no torch; tables are numpy so that a step
gathers the rows of its requests in one vectorised copy.
"""

from __future__ import annotations

from collections.abc import Hashable, Iterable, Mapping, Sequence
from dataclasses import dataclass

import numpy as np

NO_PAGE = -1


class CacheCapacityFull(Exception):
    """Not enough free pages (or slots) to hold what a step needs; nothing was changed."""

    is_capacity_error = True


class DoubleFreeError(ValueError):
    """A page was freed twice, or by a request that does not own it."""


class PageAllocator:
    """Owns every page of one pool exactly once: free list (LIFO) plus owner map."""

    def __init__(self, num_pages: int, page_size: int) -> None:
        if num_pages < 1:
            raise ValueError("num_pages must be positive")
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.total_pages = int(num_pages)
        self.page_size = int(page_size)
        self._free: list[int] = list(range(num_pages - 1, -1, -1))
        self._owner: dict[int, Hashable] = {}
        self.allocations_total = 0  # pages handed out since the start (reuse shows as > total)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return len(self._owner)

    def pages_for(self, tokens: int) -> int:
        if tokens < 0:
            raise ValueError("tokens must be non-negative")
        return -(-tokens // self.page_size)

    def can_satisfy(self, count: int) -> bool:
        return count <= len(self._free)

    def owned_by(self, owner: Hashable) -> list[int]:
        return [page for page, who in self._owner.items() if who == owner]

    def allocate(self, owner: Hashable, count: int) -> list[int]:
        if count > len(self._free):
            raise CacheCapacityFull(f"requested {count} pages, only {len(self._free)} free")
        pages = [self._free.pop() for _ in range(count)]
        self.allocations_total += count
        for page in pages:
            self._owner[page] = owner
        return pages

    def free(self, pages: Sequence[int], owner: Hashable) -> None:
        if len(set(pages)) != len(pages):
            raise DoubleFreeError("same page freed twice in one call")
        for page in pages:
            actual = self._owner.get(page)
            if actual is None:
                raise DoubleFreeError(f"page {page} is already free")
            if actual != owner:
                raise DoubleFreeError(f"page {page} owned by {actual!r}, freed by {owner!r}")
        for page in pages:
            del self._owner[page]
            self._free.append(page)

    def assert_invariants(self) -> None:
        assert len(self._owner) + len(self._free) == self.total_pages, "page lost or duplicated"
        assert len(set(self._free)) == len(self._free), "page on the free list twice"
        assert not set(self._free) & set(self._owner), "page both free and owned"
        assert all(0 <= page < self.total_pages for page in self._free)
        assert all(0 <= page < self.total_pages for page in self._owner)


@dataclass(frozen=True)
class GroupSpec:
    """One group of layers: ``window`` 0 keeps all keys; ``bytes_per_token`` is what one
    token costs over all layers of the group (used only to split a byte budget)."""

    name: str
    window: int = 0
    bytes_per_token: int = 0


class _Group:
    def __init__(self, spec: GroupSpec, num_pages: int, page_size: int, max_slots: int, width: int):
        self.spec = spec
        self.allocator = PageAllocator(num_pages, page_size)
        self.tables: dict[Hashable, list[int]] = {}
        self.host_table = np.full((max_slots, width), NO_PAGE, dtype=np.int32)

    def first_needed_page(self, start_pos: int) -> int:
        """Index of the first page a query at ``start_pos`` can still read."""
        if self.spec.window <= 0:
            return 0
        return max(0, start_pos - self.spec.window + 1) // self.allocator.page_size


class CacheManager:
    def __init__(
        self,
        groups: Sequence[GroupSpec],
        page_size: int,
        pages_per_group: Sequence[int] | int,
        max_requests: int,
        max_tokens_per_request: int,
    ) -> None:
        if not groups:
            groups = (GroupSpec("none"),)
        if isinstance(pages_per_group, int):
            pages_per_group = [pages_per_group] * len(groups)
        if len(pages_per_group) != len(groups):
            raise ValueError("pages_per_group must give one count per group")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.table_width = -(-int(max_tokens_per_request) // self.page_size)
        self.groups = [
            _Group(spec, count, self.page_size, self.max_requests, self.table_width)
            for spec, count in zip(groups, pages_per_group, strict=True)
        ]
        self._slot_of: dict[Hashable, int] = {}
        self._free_slots: list[int] = list(range(self.max_requests - 1, -1, -1))
        self._length: dict[Hashable, int] = {}
        self._dirty_slots: list[int] = []

    # ------------------------------------------------------------ admission
    def admit(self, request_id: Hashable) -> int:
        """Gives the request an empty table in every group and a state slot; returns the slot."""
        if request_id in self._slot_of:
            raise ValueError(f"request {request_id!r} is already admitted")
        if not self._free_slots:
            raise CacheCapacityFull(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        self._slot_of[request_id] = slot
        self._length[request_id] = 0
        for group in self.groups:
            group.tables[request_id] = []
            group.host_table[slot, :] = NO_PAGE
        self._dirty_slots.append(slot)
        return slot

    def is_admitted(self, request_id: Hashable) -> bool:
        return request_id in self._slot_of

    def slot(self, request_id: Hashable) -> int:
        return self._slot_of[request_id]

    def take_dirty_slots(self) -> list[int]:
        """Slots admitted since the last call; their per-request state must be zeroed."""
        dirty, self._dirty_slots = self._dirty_slots, []
        return dirty

    def release(self, request_id: Hashable) -> None:
        """Gives back every page and the slot.  Releasing an unknown request is a no-op."""
        if request_id not in self._slot_of:
            return
        slot = self._slot_of.pop(request_id)
        for group in self.groups:
            table = group.tables.pop(request_id)
            held = [page for page in table if page != NO_PAGE]
            if held:
                group.allocator.free(held, request_id)
            group.host_table[slot, :] = NO_PAGE
        self._length.pop(request_id, None)
        if slot in self._dirty_slots:
            self._dirty_slots.remove(slot)
        self._free_slots.append(slot)

    # ------------------------------------------------------------ growth
    def ensure_capacity_batch(self, required: Mapping[Hashable, tuple[int, int] | int]) -> None:
        """Grows the tables so that each request can hold positions [start, end).

        ``required[id]`` is ``(start_pos, end_pos)`` or just ``end_pos`` (start = committed
        length).  Either every page needed in every group is acquired, or
        ``CacheCapacityFull`` is raised and nothing has changed.
        """
        plan: list[tuple[_Group, Hashable, int]] = []
        for group in self.groups:
            total = 0
            for request_id, span in required.items():
                if request_id not in self._slot_of:
                    raise KeyError(f"request {request_id!r} has no block table")
                end = span[1] if isinstance(span, tuple) else int(span)
                if end > self.table_width * self.page_size:
                    raise ValueError(
                        f"request {request_id!r} needs {end} tokens; tables hold at most "
                        f"{self.table_width * self.page_size}"
                    )
                needed = group.allocator.pages_for(end)
                extra = max(0, needed - len(group.tables[request_id]))
                if extra:
                    plan.append((group, request_id, extra))
                    total += extra
            if not group.allocator.can_satisfy(total):
                raise CacheCapacityFull(
                    f"group {group.spec.name!r}: need {total} more pages, "
                    f"{group.allocator.free_count} free"
                )
        for group, request_id, extra in plan:
            pages = group.allocator.allocate(request_id, extra)
            table = group.tables[request_id]
            first = len(table)
            table.extend(pages)
            group.host_table[self._slot_of[request_id], first:first + extra] = pages

    def commit_lengths(self, lengths: Mapping[Hashable, int]) -> None:
        """Records that the step ran, and gives back pages that fell out of a window."""
        for request_id, length in lengths.items():
            for group in self.groups:
                if group.allocator.pages_for(length) > len(group.tables[request_id]):
                    raise RuntimeError(f"length {length} exceeds the table of {request_id!r}")
            self._length[request_id] = max(self._length[request_id], int(length))
            self._retire_behind_window(request_id)

    def _retire_behind_window(self, request_id: Hashable) -> None:
        length = self._length[request_id]
        slot = self._slot_of[request_id]
        for group in self.groups:
            if group.spec.window <= 0:
                continue
            table = group.tables[request_id]
            # the next query sits at position `length`; it reads keys >= length - window + 1
            keep_from = group.first_needed_page(length)
            retired = [table[i] for i in range(min(keep_from, len(table))) if table[i] != NO_PAGE]
            if retired:
                group.allocator.free(retired, request_id)
                for index in range(min(keep_from, len(table))):
                    table[index] = NO_PAGE
                group.host_table[slot, :keep_from] = NO_PAGE

    # ------------------------------------------------------------ queries
    def committed_length(self, request_id: Hashable) -> int:
        return self._length[request_id]

    def allocated_tokens(self, request_id: Hashable) -> int:
        if request_id not in self._slot_of:
            return 0
        return max(
            sum(1 for page in group.tables[request_id] if page != NO_PAGE) for group in self.groups
        ) * self.page_size

    def block_table(self, request_id: Hashable, group: int = 0) -> list[int]:
        return list(self.groups[group].tables[request_id])

    def table_rows(self, group: int, slots: np.ndarray, width: int) -> np.ndarray:
        """Block-table rows of the given slots, ``width`` entries each (int32, -1 = no page)."""
        return self.groups[group].host_table[slots, :width]

    def width_for(self, max_end_pos: int) -> int:
        return max(1, -(-max_end_pos // self.page_size))

    def live_requests(self) -> Iterable[Hashable]:
        return tuple(self._slot_of)

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].allocator.free_count

    def total_pages(self, group: int = 0) -> int:
        return self.groups[group].allocator.total_pages

    def stats(self) -> dict[str, object]:
        per_group = []
        for group in self.groups:
            alloc = group.allocator
            per_group.append(
                dict(
                    name=group.spec.name,
                    window=group.spec.window,
                    pages_total=alloc.total_pages,
                    pages_used=alloc.used_count,
                    pages_free=alloc.free_count,
                    utilization=round(alloc.used_count / alloc.total_pages, 4),
                )
            )
        return dict(
            kind="paged",
            page_size=self.page_size,
            requests=len(self._slot_of),
            slots_free=len(self._free_slots),
            groups=per_group,
            blocks_total=per_group[0]["pages_total"],
            blocks_used=per_group[0]["pages_used"],
        )

    def assert_invariants(self) -> None:
        assert len(self._free_slots) + len(self._slot_of) == self.max_requests, "slot lost"
        assert len(set(self._free_slots)) == len(self._free_slots), "slot free twice"
        assert len(set(self._slot_of.values())) == len(self._slot_of), "slot held twice"
        for group in self.groups:
            group.allocator.assert_invariants()
            held: list[int] = []
            for request_id, table in group.tables.items():
                assert request_id in self._slot_of
                pages = [page for page in table if page != NO_PAGE]
                held.extend(pages)
                assert sorted(pages) == sorted(group.allocator.owned_by(request_id)), (
                    "table and owner map disagree"
                )
                row = group.host_table[self._slot_of[request_id]]
                assert list(row[: len(table)]) == table, "host mirror out of date"
                assert (row[len(table):] == NO_PAGE).all(), "stale entries in host mirror"
            assert len(set(held)) == len(held), "page held twice"
            assert len(held) == group.allocator.used_count, "owned page in no table"
