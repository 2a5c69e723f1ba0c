"""Device memory behind the cache manager: pages of keys and values per group and the
per-request state tensors.  The reference's counterpart is `PagedKVCache`
(kv/cache.py:13-26): K and V as [layers, pages, page_size, kv_heads, head_dim], zero-filled; here
the kv head comes before the offset in the page, so that the keys a thread block streams (one
kv head) lie in runs of page_size * head_dim elements instead of head_dim."""

from __future__ import annotations

import torch

from ..parts.base import CacheNeed, StateNeed
from ..parts.context import LaneView
from .manager import CacheManager


class CacheStorage:
    def __init__(self, manager: CacheManager, lane_needs: list[tuple[CacheNeed | None, StateNeed | None]],
                 dtype: torch.dtype, device: torch.device) -> None:
        self.manager = manager
        self.dtype, self.device = dtype, device
        self.group_kv: list[torch.Tensor] = []
        for g in manager.groups:
            s = g.spec
            # [lane in group, k|v, page, kv head, offset, dim]: one kv head's tokens of a page are contiguous
            self.group_kv.append(torch.zeros((len(s.lanes), 2, manager.num_blocks, s.kv_heads, s.page_size, s.head_dim),
                                             dtype=dtype, device=device))
        self.state: dict[int, torch.Tensor] = {}
        for lane, (_, st) in enumerate(lane_needs):
            if st is not None:
                # one slot more than requests can hold: the scratch slot that a step's padding rows point at
                self.state[lane] = torch.zeros((manager.slots.num_slots + 1, *st.shape), dtype=st.dtype, device=device)
        self.lane_needs = lane_needs

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.group_kv) + \
            sum(t.numel() * t.element_size() for t in self.state.values())

    def lane_views(self, group_tables: list[torch.Tensor | None]) -> list[LaneView]:
        """`group_tables[g]`: this step's device block table of group g."""
        views = []
        for lane, (need, st) in enumerate(self.lane_needs):
            gi = self.manager.lane_group[lane]
            if gi is None:
                views.append(LaneView(None, None, None, self.manager.block_size, 0, self.state.get(lane)))
                continue
            spec = self.manager.groups[gi].spec
            idx = spec.lanes.index(lane)
            kv = self.group_kv[gi][idx]
            views.append(LaneView(kv[0], kv[1], group_tables[gi], spec.page_size, spec.window, self.state.get(lane)))
        return views

    def zero_state_slots(self, slots: list[int]) -> None:
        if not slots or not self.state:
            return
        idx = torch.tensor(slots, dtype=torch.int64, device=self.device)
        for t in self.state.values():
            t.index_fill_(0, idx, 0)
