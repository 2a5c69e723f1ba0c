"""Names shared by the cache manager and its users: the geometry of a cache group, the error for
a pool that has run out, and the mark of a released table entry.  No tensors.

The allocator itself (free lists, block tables, state slots) is native code, csrc/host_cache.cu;
`manager.py` is its Python face.
"""

from __future__ import annotations

from dataclasses import dataclass


class PoolExhausted(Exception):
    """Not enough free pages, or no free state slot; nothing was changed."""


@dataclass(frozen=True)
class GroupSpec:
    """Cache lanes that share one geometry, one pool and one block table per request."""

    lanes: tuple[int, ...]
    kv_heads: int
    head_dim: int
    page_size: int
    window: int = 0  # 0: every position is kept; w > 0: a query reads the last w positions only

    def blocks_for(self, seq_len: int) -> int:
        return -(-seq_len // self.page_size)

    def first_needed_block(self, seq_len: int) -> int:
        """First logical block that a query at position >= seq_len can still read."""
        if self.window <= 0:
            return 0
        return max(0, seq_len - self.window + 1) // self.page_size

    def peak_pages(self, total_len: int, longest_portion: int) -> int:
        """Most pages one request can hold at any time on its way to `total_len` positions
        when no step brings more than `longest_portion` of its tokens."""
        full = self.blocks_for(total_len)
        if self.window <= 0:
            return full
        span = self.window - 1 + max(1, longest_portion)
        return min(full, self.blocks_for(span) + 1)


RELEASED = -1  # block-table entry of a page that a window has passed
