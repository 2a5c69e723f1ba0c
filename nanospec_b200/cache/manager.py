"""The cache manager: which pages and which state slot each live request holds.

One `CacheManager` serves all cache lanes of a model.  Lanes with the same geometry (kv
heads, head size, window) form a group with its own page pool and its own block table per
request.  A request's life: `begin` (state slot, empty tables) -> `extend` before each step
that brings tokens (pages for the new positions, in every group, or `PoolExhausted` with
nothing changed) -> `trim` after the step (pages that a window has passed go back) -> `end`
(everything goes back).  `rollback` shortens a request and returns whole pages past the new
end (kv/allocator.py:61-69 in the reference).

The free lists, tables and slots live in native code (csrc/host_cache.cu), which also lays a
step's description out for the device in one call (`pack_step`, `pack_decode`); this class is its
face: it turns status codes into exceptions and keeps what is pure arithmetic (how many pages a
length needs) in Python, where the scheduler asks for it many times per step.
"""

from __future__ import annotations

import ctypes
from collections.abc import Mapping
from ctypes import POINTER, byref, c_int, c_longlong, c_void_p

from ..ops import lib
from ..parts.base import CacheNeed, StateNeed
from .pages import RELEASED, GroupSpec, PoolExhausted  # noqa: F401  (RELEASED is part of this module's surface)

_EXHAUSTED, _NOT_LIVE, _SMALL, _INVARIANT = 4, 5, 6, 7
_P, _I, _L = c_void_p, c_int, c_longlong
_PI, _PL = POINTER(c_int), POINTER(c_longlong)

_SIGNATURES = {
    "ns_cache_create": [_I, _PI, _PI, _I, _I, POINTER(c_void_p)],
    "ns_cache_destroy": [_P],
    "ns_cache_begin": [_P, _L],
    "ns_cache_extend": [_P, _L, _L],
    "ns_cache_trim": [_P, _L, _PI],
    "ns_cache_trim_many": [_P, _I, _P],
    "ns_cache_rollback": [_P, _L, _L],
    "ns_cache_end": [_P, _L],
    "ns_cache_need": [_P, _L, _L, _PI],
    "ns_cache_free_pages": [_P, _PI],
    "ns_cache_held_pages": [_P, _L, _PI],
    "ns_cache_lookup": [_P, _L, _PL, _PI],
    "ns_cache_counts": [_P, _PI, _PI, _PI],
    "ns_cache_live": [_P, _PL, _I],
    "ns_cache_table": [_P, _I, _L, _PI, _I, _PI, _PI],
    "ns_cache_free_list": [_P, _I, _PI, _I],
    "ns_cache_take_fresh": [_P, _PI, _I],
    "ns_cache_check": [_P],
    "ns_step_pack": [_P, _I, _P, _P, _P, _I, _P, _I, _P, _P, _I, _P, _PI, _L, _P, _L, _PI, _PI, _PL, _PL, _PI, _PL],
    "ns_step_pack_decode": [_P, _I, _I, _P, _L, _I, _P, _I, _I, _I, _I, _PI, _I, _I, _I],
}
_declared = False


def _native():
    global _declared
    if not _declared:
        for name, sig in _SIGNATURES.items():
            lib.declare(name, sig)
        _declared = True
    return lib.load()


class _Pool:
    """One group's pool as its users see it."""

    def __init__(self, manager: "CacheManager", group: int, num_pages: int) -> None:
        self._m, self._g, self.num_pages = manager, group, num_pages

    @property
    def num_free(self) -> int:
        return self._m.free_pages()[self._g]

    def free_pages(self) -> list[int]:
        """The free list, the page that goes out next last."""
        buf = (c_int * self.num_pages)()
        self._m._call("ns_cache_free_list", self._g, buf, self.num_pages)
        return list(buf[: self.num_free])


class CacheGroup:
    def __init__(self, manager: "CacheManager", index: int, spec: GroupSpec, num_pages: int) -> None:
        self.spec = spec
        self.pool = _Pool(manager, index, num_pages)

    def blocks_for(self, seq_len: int) -> int:
        return self.spec.blocks_for(seq_len)

    def first_needed_block(self, seq_len: int) -> int:
        return self.spec.first_needed_block(seq_len)

    def peak_pages(self, total_len: int, longest_portion: int) -> int:
        return self.spec.peak_pages(total_len, longest_portion)


class _Slots:
    def __init__(self, manager: "CacheManager", num_slots: int) -> None:
        self._m, self.num_slots = manager, num_slots

    @property
    def num_free(self) -> int:
        return self._m._counts()[1]


class _SeqLens(Mapping):
    """`manager.seq_len[request]`: positions the request holds; iterates over the live requests in the order
    in which they began."""

    def __init__(self, manager: "CacheManager") -> None:
        self._m = manager

    def __getitem__(self, req_id: int) -> int:
        n = self._m._lookup(req_id)[0]
        if n < 0:
            raise KeyError(req_id)
        return n

    def __contains__(self, req_id) -> bool:
        return isinstance(req_id, int) and self._m._lookup(req_id)[0] >= 0

    def __iter__(self):
        return iter(self._m.live)

    def __len__(self) -> int:
        return self._m._counts()[0]


class CacheManager:
    def __init__(self, lane_needs: list[tuple[CacheNeed | None, StateNeed | None]], num_blocks: int, block_size: int,
                 num_state_slots: int) -> None:
        if num_blocks <= 0 or block_size <= 0 or num_state_slots <= 0:
            raise ValueError("a cache needs at least one page, a positive page size and one state slot")
        self.block_size = block_size
        self.num_blocks = num_blocks
        by_geometry: dict[tuple[int, int, int], list[int]] = {}
        for lane, (need, _) in enumerate(lane_needs):
            if need is not None:
                by_geometry.setdefault((need.kv_heads, need.head_dim, need.window), []).append(lane)
        specs = [GroupSpec(tuple(lanes), kvh, hd, block_size, window) for (kvh, hd, window), lanes in by_geometry.items()]
        self._lib = _native()
        n = len(specs)
        handle = c_void_p()
        self._n_groups = n
        self._status(self._lib.ns_cache_create(n, (c_int * max(n, 1))(*[s.page_size for s in specs]),
                                               (c_int * max(n, 1))(*[s.window for s in specs]), num_blocks, num_state_slots,
                                               byref(handle)))
        self._h = handle
        self.groups: list[CacheGroup] = [CacheGroup(self, gi, s, num_blocks) for gi, s in enumerate(specs)]
        self.lane_group: list[int | None] = [None] * len(lane_needs)
        for gi, g in enumerate(self.groups):
            for lane in g.spec.lanes:
                self.lane_group[lane] = gi
        self.state_lanes = [lane for lane, (_, st) in enumerate(lane_needs) if st is not None]
        self.slots = _Slots(self, num_state_slots)
        self.seq_len = _SeqLens(self)
        self._ints = (c_int * max(n, 1))()

    def __del__(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        try:
            if h:
                self._lib.ns_cache_destroy(h)
        except Exception:  # the interpreter is shutting down and the library is gone: the process's memory goes with it
            pass

    # ---- native calls ---------------------------------------------------------------------
    def _status(self, status: int) -> None:
        if status == 0:
            return
        text = self._lib.ns_last_error().decode(errors="replace")
        if status == _EXHAUSTED:
            raise PoolExhausted(text)
        if status == _NOT_LIVE:
            raise KeyError(text)
        if status == _INVARIANT:
            raise AssertionError(text)
        raise ValueError(text)

    def _call(self, name: str, *args) -> None:
        self._status(getattr(self._lib, name)(self._h, *args))

    def _lookup(self, req_id: int) -> tuple[int, int]:
        n, slot = c_longlong(), c_int()
        self._call("ns_cache_lookup", req_id, byref(n), byref(slot))
        return n.value, slot.value

    def _counts(self) -> tuple[int, int, int]:
        a, b, c = c_int(), c_int(), c_int()
        self._call("ns_cache_counts", byref(a), byref(b), byref(c))
        return a.value, b.value, c.value

    # ---- queries ------------------------------------------------------------------------
    @property
    def live(self) -> list[int]:
        n = self._counts()[0]
        buf = (c_longlong * max(n, 1))()
        self._call("ns_cache_live", buf, n)
        return list(buf[:n])

    def free_pages(self) -> list[int]:
        self._call("ns_cache_free_pages", self._ints)
        return list(self._ints[: self._n_groups])

    def need(self, req_id: int | None, new_len: int) -> list[int]:
        """Per group: pages to take so that the request (None: a new one) reaches new_len."""
        self._call("ns_cache_need", -1 if req_id is None else req_id, new_len, self._ints)
        return list(self._ints[: self._n_groups])

    def need_between(self, cur_len: int, new_len: int) -> list[int]:
        """The same by arithmetic alone, for a live request that holds `cur_len` positions (a request's tables
        are always exactly as long as its length needs): what the scheduler asks for every request and step."""
        return [g.spec.blocks_for(new_len) - g.spec.blocks_for(cur_len) for g in self.groups]

    def peak_pages(self, total_len: int, longest_portion: int) -> list[int]:
        return [g.peak_pages(total_len, longest_portion) for g in self.groups]

    def held_pages(self, req_id: int) -> list[int]:
        self._call("ns_cache_held_pages", req_id, self._ints)
        return list(self._ints[: self._n_groups])

    def can_extend(self, req_id: int | None, n_tokens: int) -> bool:
        cur = self.seq_len.get(req_id, 0) if req_id is not None else 0
        return all(n <= f for n, f in zip(self.need(req_id, cur + n_tokens), self.free_pages()))

    def table(self, group: int, req_id: int) -> list[int]:
        cap = self.groups[group].spec.blocks_for(max(1, self.seq_len[req_id]))
        buf = (c_int * cap)()
        n, first = c_int(), c_int()
        self._call("ns_cache_table", group, req_id, buf, cap, byref(n), byref(first))
        return list(buf[: n.value])

    def state_slot(self, req_id: int) -> int:
        n, slot = self._lookup(req_id)
        if n < 0:
            raise KeyError(req_id)
        return slot

    @property
    def scratch_slot(self) -> int:
        """The state slot that no request ever holds: padding rows of a step carry it, so that a mixer
        which reads and writes state by `state_slot` on the device needs no mask for them."""
        return self.slots.num_slots

    # ---- life of a request ----------------------------------------------------------------
    def begin(self, req_id: int) -> None:
        self._call("ns_cache_begin", req_id)

    def extend(self, req_id: int, n_tokens: int) -> None:
        """Makes room for n_tokens more positions in every group, or raises PoolExhausted
        and leaves everything as it was."""
        self._call("ns_cache_extend", req_id, n_tokens)

    def trim(self, req_id: int) -> int:
        """After a step: gives back the pages that no later query of this request can read
        (those wholly behind a group's window).  Returns the number of pages released."""
        released = c_int()
        self._call("ns_cache_trim", req_id, byref(released))
        return released.value

    def trim_many(self, req_ids) -> None:
        """`trim` for every request of a step in one call; `req_ids`: a ctypes or numpy array of int64."""
        self._call("ns_cache_trim_many", len(req_ids), req_ids.ctypes.data if hasattr(req_ids, "ctypes") else req_ids)

    def rollback(self, req_id: int, seq_len: int) -> None:
        self._call("ns_cache_rollback", req_id, seq_len)

    def end(self, req_id: int) -> None:
        self._call("ns_cache_end", req_id)

    def take_fresh_slots(self) -> list[int]:
        """State slots handed out since the last call: their state must be zeroed before the next step."""
        n = self._counts()[2]
        if n == 0:
            return []
        buf = (c_int * n)()
        self._call("ns_cache_take_fresh", buf, n)
        return list(buf)

    # ---- a step's description ----------------------------------------------------------------
    def pack_step(self, req_ids, q_lens, tokens, want_rows, take_dst, take_src, extra, tile_q: tuple[int, int],
                  max_positions: int, buf, cap: int):
        """Reserves pages for every entry (all or none) and writes the step's description into `buf` (an int32
        numpy array of `cap` entries): see ns_step_pack in csrc/host_cache.cu for the layout.  The arguments are
        contiguous numpy arrays (int64 ids, int32 the rest; `extra` is copied along as it is).  Returns (offsets,
        table widths, counts, total, longest portion, longest sequence) with counts = (one-token requests, query
        tiles of tile_q[0], of tile_q[1], longest sequence among the one-token requests, items of the decode work
        list, slots of scratch it needs); raises BufferError with the ints needed when `buf` is too small (nothing
        changed)."""
        G = self._n_groups
        offsets, widths, counts = (c_int * (14 + G))(), (c_int * max(G, 1))(), (c_longlong * 6)()
        total, max_q, max_kv = c_longlong(), c_int(), c_longlong()
        status = self._lib.ns_step_pack(
            self._h, len(req_ids), req_ids.ctypes.data, q_lens.ctypes.data, tokens.ctypes.data, len(want_rows),
            want_rows.ctypes.data, len(take_dst), take_dst.ctypes.data, take_src.ctypes.data, len(extra), extra.ctypes.data,
            (c_int * 2)(*tile_q), max_positions, buf.ctypes.data, cap, offsets, widths, counts, byref(total), byref(max_q),
            byref(max_kv))
        if status == _SMALL:
            raise BufferError(total.value)
        self._status(status)
        return list(offsets), list(widths[:G]), list(counts), total.value, max_q.value, max_kv.value

    def pack_decode(self, req_ids, size: int, max_positions: int, buf, off: dict[str, int], table_off, width: int,
                    n_work: int = 0) -> None:
        """The description of a decode-only step padded to a graph bucket of `size` rows (ns_step_pack_decode); with
        `n_work` also the decode attention kernel's work list of that many items at off["work"]."""
        self._status(self._lib.ns_step_pack_decode(
            self._h, len(req_ids), size, req_ids.ctypes.data, max_positions, self.scratch_slot, buf.ctypes.data,
            off["positions"], off["token_req"], off["kv_len"], off["slots"], table_off, width,
            off.get("work", 0) if n_work else 0, n_work))

    # ---- invariants ---------------------------------------------------------------------
    def check(self) -> None:
        """No page lost, held twice or freed twice; tables as long as their sequences need; every slot in one place."""
        self._call("ns_cache_check")
