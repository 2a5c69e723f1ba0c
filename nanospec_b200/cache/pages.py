"""Pages and block tables, host side.  No tensors.

Follows the behaviour of the reference's `BlockAllocator` (kv/allocator.py:22-85): a LIFO
free list that hands out page 0 first and reuses the most recently freed page first; a block
table per request; exhaustion is raised before anything is changed; `check()` asserts that
every page is in exactly one place.  Added here: several cache groups, each with a pool and
tables of its own, and groups that only need a window of the most recent positions and give
the pages behind it back while the request is still running.
"""

from __future__ import annotations

from dataclasses import dataclass, field


class PoolExhausted(Exception):
    """Not enough free pages; nothing was changed."""


class PagePool:
    """Free list of page numbers 0..num_pages-1."""

    def __init__(self, num_pages: int) -> None:
        if num_pages <= 0:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() hands out page 0 first
        self._is_free = [True] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> list[int]:
        if n > len(self._free):
            raise PoolExhausted(f"need {n} pages, {len(self._free)} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._is_free[p] = False
        return out

    def give(self, pages: list[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or self._is_free[p]:
                raise AssertionError(f"page {p} freed twice or never handed out")
            self._is_free[p] = True
            self._free.append(p)

    def free_pages(self) -> list[int]:
        return list(self._free)


@dataclass(frozen=True)
class GroupSpec:
    """Cache lanes that share one geometry, one pool and one block table per request."""

    lanes: tuple[int, ...]
    kv_heads: int
    head_dim: int
    page_size: int
    window: int = 0  # 0: every position is kept; w > 0: a query reads the last w positions only


RELEASED = -1  # block-table entry of a page that a window has passed


@dataclass
class GroupTable:
    pages: list[int] = field(default_factory=list)  # one entry per logical block, RELEASED once given back
    first_live: int = 0                             # blocks before this index are released


class CacheGroup:
    def __init__(self, spec: GroupSpec, num_pages: int) -> None:
        self.spec = spec
        self.pool = PagePool(num_pages)
        self.tables: dict[int, GroupTable] = {}

    def blocks_for(self, seq_len: int) -> int:
        return -(-seq_len // self.spec.page_size)

    def first_needed_block(self, seq_len: int) -> int:
        """First logical block that a query at position >= seq_len can still read."""
        if self.spec.window <= 0:
            return 0
        first_pos = seq_len - self.spec.window + 1
        return max(0, first_pos) // self.spec.page_size

    def need(self, req_id: int | None, new_len: int) -> int:
        """Pages that must be taken from the pool to hold positions up to new_len."""
        have = len(self.tables[req_id].pages) if req_id is not None and req_id in self.tables else 0
        return max(0, self.blocks_for(new_len) - have)

    def peak_pages(self, total_len: int, longest_portion: int) -> int:
        """Most pages one request can hold at any time on its way to `total_len` positions
        when no step brings more than `longest_portion` of its tokens."""
        full = self.blocks_for(total_len)
        if self.spec.window <= 0:
            return full
        span = self.spec.window - 1 + max(1, longest_portion)
        return min(full, self.blocks_for(span) + 1)

    def live_pages(self, req_id: int) -> int:
        t = self.tables[req_id]
        return len(t.pages) - t.first_live


class SlotPool:
    """Slots of fixed-size per-request state (LIFO, slot 0 first)."""

    def __init__(self, num_slots: int) -> None:
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self.owner: dict[int, int] = {}  # req_id -> slot

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self, req_id: int) -> int:
        if req_id in self.owner:
            raise AssertionError(f"request {req_id} already holds state slot {self.owner[req_id]}")
        if not self._free:
            raise PoolExhausted("no free state slot")
        slot = self._free.pop()
        self.owner[req_id] = slot
        return slot

    def release(self, req_id: int) -> int:
        slot = self.owner.pop(req_id)
        self._free.append(slot)
        return slot

    def check(self) -> None:
        seen = sorted(self._free + list(self.owner.values()))
        assert seen == list(range(self.num_slots)), "state slot lost or held twice"
