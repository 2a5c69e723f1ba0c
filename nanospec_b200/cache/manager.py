"""The cache manager: which pages and which state slot each live request holds.

One `CacheManager` serves all cache lanes of a model.  Lanes with the same geometry (kv
heads, head size, window) form a group with its own page pool and its own block table per
request.  A request's life: `begin` (state slot, empty tables) -> `extend` before each step
that brings tokens (pages for the new positions, in every group, or `PoolExhausted` with
nothing changed) -> `trim` after the step (pages that a window has passed go back) -> `end`
(everything goes back).  `rollback` shortens a request and returns whole pages past the new
end (kv/allocator.py:61-69 in the reference).
"""

from __future__ import annotations

from ..parts.base import CacheNeed, StateNeed
from .pages import RELEASED, CacheGroup, GroupSpec, GroupTable, PagePool, PoolExhausted, SlotPool


class CacheManager:
    def __init__(self, lane_needs: list[tuple[CacheNeed | None, StateNeed | None]], num_blocks: int, block_size: int,
                 num_state_slots: int) -> None:
        self.block_size = block_size
        self.num_blocks = num_blocks
        by_geometry: dict[tuple[int, int, int], list[int]] = {}
        for lane, (need, _) in enumerate(lane_needs):
            if need is not None:
                by_geometry.setdefault((need.kv_heads, need.head_dim, need.window), []).append(lane)
        self.groups: list[CacheGroup] = [
            CacheGroup(GroupSpec(tuple(lanes), kvh, hd, block_size, window), num_blocks)
            for (kvh, hd, window), lanes in by_geometry.items()]
        self.lane_group: list[int | None] = [None] * len(lane_needs)
        for gi, g in enumerate(self.groups):
            for lane in g.spec.lanes:
                self.lane_group[lane] = gi
        self.state_lanes = [lane for lane, (_, st) in enumerate(lane_needs) if st is not None]
        self.slots = SlotPool(num_state_slots)
        self.seq_len: dict[int, int] = {}
        self.fresh_slots: list[int] = []  # slots handed out since the last step: their state must be zeroed

    # ---- queries ------------------------------------------------------------------------
    @property
    def live(self) -> list[int]:
        return list(self.seq_len)

    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    def need(self, req_id: int | None, new_len: int) -> list[int]:
        """Per group: pages to take so that the request (None: a new one) reaches new_len."""
        return [g.need(req_id, new_len) for g in self.groups]

    def peak_pages(self, total_len: int, longest_portion: int) -> list[int]:
        return [g.peak_pages(total_len, longest_portion) for g in self.groups]

    def held_pages(self, req_id: int) -> list[int]:
        return [g.live_pages(req_id) for g in self.groups]

    def can_extend(self, req_id: int | None, n_tokens: int) -> bool:
        cur = self.seq_len.get(req_id, 0) if req_id is not None else 0
        return all(n <= g.pool.num_free for n, g in zip(self.need(req_id, cur + n_tokens), self.groups))

    def table(self, group: int, req_id: int) -> list[int]:
        return self.groups[group].tables[req_id].pages

    def state_slot(self, req_id: int) -> int:
        return self.slots.owner[req_id]

    @property
    def scratch_slot(self) -> int:
        """The state slot that no request ever holds: padding rows of a step carry it, so that a mixer
        which reads and writes state by `state_slot` on the device needs no mask for them."""
        return self.slots.num_slots

    # ---- life of a request ----------------------------------------------------------------
    def begin(self, req_id: int) -> None:
        if req_id in self.seq_len:
            raise AssertionError(f"request {req_id} is already live")
        slot = self.slots.acquire(req_id)  # raises PoolExhausted before anything else changes
        self.fresh_slots.append(slot)
        for g in self.groups:
            g.tables[req_id] = GroupTable()
        self.seq_len[req_id] = 0

    def extend(self, req_id: int, n_tokens: int) -> None:
        """Makes room for n_tokens more positions in every group, or raises PoolExhausted
        and leaves everything as it was."""
        new_len = self.seq_len[req_id] + n_tokens
        needs = self.need(req_id, new_len)
        for n, g in zip(needs, self.groups):
            if n > g.pool.num_free:
                raise PoolExhausted(f"request {req_id} needs {n} pages, {g.pool.num_free} free")
        for n, g in zip(needs, self.groups):
            g.tables[req_id].pages.extend(g.pool.take(n))
        self.seq_len[req_id] = new_len

    def trim(self, req_id: int) -> int:
        """After a step: gives back the pages that no later query of this request can read
        (those wholly behind a group's window).  Returns the number of pages released."""
        released = 0
        length = self.seq_len[req_id]
        for g in self.groups:
            t = g.tables[req_id]
            first = min(g.first_needed_block(length), len(t.pages))
            if first > t.first_live:
                back = [p for p in t.pages[t.first_live:first]]
                g.pool.give(back)
                for i in range(t.first_live, first):
                    t.pages[i] = RELEASED
                t.first_live = first
                released += len(back)
        return released

    def rollback(self, req_id: int, seq_len: int) -> None:
        if not 0 <= seq_len <= self.seq_len[req_id]:
            raise AssertionError("rollback goes backwards only")
        for g in self.groups:
            t = g.tables[req_id]
            keep = g.blocks_for(seq_len)
            if keep < t.first_live:
                raise AssertionError("cannot roll back behind pages that a window has already released")
            g.pool.give(t.pages[keep:])
            del t.pages[keep:]
        self.seq_len[req_id] = seq_len

    def end(self, req_id: int) -> None:
        for g in self.groups:
            t = g.tables.pop(req_id)
            g.pool.give([p for p in t.pages if p != RELEASED])
        self.slots.release(req_id)
        del self.seq_len[req_id]

    def take_fresh_slots(self) -> list[int]:
        out, self.fresh_slots = self.fresh_slots, []
        return out

    # ---- invariants ---------------------------------------------------------------------
    def check(self) -> None:
        """No page lost, held twice or freed twice; tables as long as their sequences need."""
        for g in self.groups:
            seen = g.pool.free_pages()
            for rid, t in g.tables.items():
                assert rid in self.seq_len
                assert len(t.pages) == g.blocks_for(self.seq_len[rid]), (t.pages, self.seq_len[rid])
                assert all(p == RELEASED for p in t.pages[:t.first_live])
                live = t.pages[t.first_live:]
                assert all(p != RELEASED for p in live)
                seen.extend(live)
            assert sorted(seen) == list(range(g.pool.num_pages)), "page lost or held twice"
        self.slots.check()
        assert set(self.slots.owner) == set(self.seq_len)
