"""The cache manager on the host: no page lost, held twice or freed twice, under fixed and
random orders of requests; windows give pages back early; exhaustion changes nothing; state
slots (no GPU).  The behaviours of the reference's allocator tests are kept
(tests/test_allocator.py there): round trip, rollback of whole pages, exhaustion leaves the
state intact, churn with a check after every operation, scattered pages."""

from __future__ import annotations

import random

import pytest

from nanospec_b200.cache import RELEASED, CacheManager, PoolExhausted
from nanospec_b200.parts import CacheNeed, StateNeed


def manager(num_blocks=8, block_size=4, lanes=2, window=0, slots=4):
    return CacheManager([(CacheNeed(2, 8, window), None)] * lanes, num_blocks, block_size, slots)


def test_round_trip_and_page_arithmetic():
    m = manager()
    m.begin(0)
    m.extend(0, 5)
    assert len(m.table(0, 0)) == 2 and m.table(0, 0) == [0, 1]  # page 0 goes out first
    m.extend(0, 3)  # exactly two full pages: no new page
    assert len(m.table(0, 0)) == 2
    m.extend(0, 1)
    assert len(m.table(0, 0)) == 3 and m.seq_len[0] == 9
    m.check()
    m.end(0)
    assert m.free_pages() == [8] and not m.live
    m.check()


def test_freed_pages_are_used_again_most_recent_first():
    m = manager()
    m.begin(0), m.extend(0, 8)
    m.begin(1), m.extend(1, 4)
    first = list(m.table(0, 0))
    m.end(0)
    m.begin(2), m.extend(2, 4)
    assert m.table(0, 2)[0] == first[-1]  # LIFO: the page freed last is handed out first
    m.check()


def test_rollback_frees_only_whole_pages_past_the_tail():
    m = manager()
    m.begin(0), m.extend(0, 10)
    pages = list(m.table(0, 0))
    m.rollback(0, 9)
    assert m.table(0, 0) == pages
    m.rollback(0, 8)
    assert m.table(0, 0) == pages[:2]
    m.rollback(0, 1)
    assert m.table(0, 0) == pages[:1] and m.free_pages() == [7]
    m.rollback(0, 0)
    assert m.table(0, 0) == [] and m.free_pages() == [8]
    m.check()


def test_exhaustion_raises_and_leaves_everything_as_it_was():
    m = manager(num_blocks=4, block_size=2)
    m.begin(0), m.extend(0, 6)
    m.begin(1)
    with pytest.raises(PoolExhausted):
        m.extend(1, 3)
    assert m.seq_len[1] == 0 and m.table(0, 1) == [] and m.free_pages() == [1]
    m.check()
    m.extend(1, 2)
    assert not m.can_extend(0, 1) and not m.can_extend(1, 1) and m.can_extend(None, 0)
    m.check()


def test_groups_by_geometry_have_pools_of_their_own():
    needs = [(CacheNeed(2, 8, 0), None), (CacheNeed(2, 8, 6), None), (CacheNeed(2, 8, 0), None), (CacheNeed(1, 16, 0), None),
             (None, StateNeed((4,)))]
    m = CacheManager(needs, num_blocks=10, block_size=4, num_state_slots=3)
    assert len(m.groups) == 3 and m.lane_group == [0, 1, 0, 2, None] and m.state_lanes == [4]
    assert m.groups[0].spec.lanes == (0, 2) and m.groups[1].spec.window == 6
    m.begin(7), m.extend(7, 9)
    assert m.free_pages() == [7, 7, 7]  # each group took its own three pages
    m.check()


def test_window_gives_pages_back_while_the_request_runs():
    m = manager(num_blocks=6, block_size=4, lanes=1, window=6)
    m.begin(0)
    m.extend(0, 9)   # a prompt portion needs all of its positions during the step
    assert m.free_pages() == [3]
    assert m.trim(0) == 1  # next query (position 9) reads 4..9: block 0 is behind the window
    assert m.table(0, 0)[0] == RELEASED and m.free_pages() == [4]
    m.check()
    for _ in range(40):  # decoding far beyond the pool's size works: pages are recycled
        m.extend(0, 1)
        m.trim(0)
        m.check()
        assert m.held_pages(0)[0] <= 3
    assert m.seq_len[0] == 49
    with pytest.raises(AssertionError):
        m.rollback(0, 3)  # behind released pages
    m.end(0)
    assert m.free_pages() == [6]
    m.check()


def test_peak_pages_for_reservation():
    full = manager(num_blocks=100, block_size=4, lanes=1)
    assert full.peak_pages(33, 8) == [9]
    win = manager(num_blocks=100, block_size=4, lanes=1, window=6)
    assert win.peak_pages(33, 8) == [5]    # window - 1 + portion = 13 positions -> 4 pages, + 1 for alignment
    assert win.peak_pages(7, 8) == [2]     # never more than the whole sequence needs


def test_double_begin_double_end_and_double_free_are_caught():
    m = manager()
    m.begin(0)
    with pytest.raises(AssertionError):
        m.begin(0)
    m.extend(0, 4)
    m.end(0)
    with pytest.raises(KeyError):
        m.end(0)
    with pytest.raises(KeyError):
        m.extend(0, 1)
    assert m.free_pages() == [8, ] and m.groups[0].pool.free_pages()[-1] == 0  # the page freed last goes out next
    m.check()


def test_state_slots():
    s = manager(slots=2)
    s.begin(10), s.begin(11)
    assert s.state_slot(10) == 0 and s.state_slot(11) == 1 and s.scratch_slot == 2
    with pytest.raises(PoolExhausted):
        s.begin(12)
    s.end(10)
    s.begin(12)
    assert s.state_slot(12) == 0 and s.slots.num_free == 0  # the slot given back last goes out next
    s.check()
    m = manager(slots=1)
    m.begin(0)
    assert m.take_fresh_slots() == [0] and m.take_fresh_slots() == []
    with pytest.raises(PoolExhausted):
        m.begin(1)
    assert 1 not in m.seq_len
    m.check()


@pytest.mark.parametrize("window", [0, 9])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_orders_keep_every_invariant(seed, window):
    rng = random.Random(seed)
    m = CacheManager([(CacheNeed(2, 8, 0), None), (CacheNeed(2, 8, window), None)], num_blocks=64, block_size=4,
                     num_state_slots=12)
    live, next_id = [], 0
    for _ in range(600):
        op = rng.random()
        try:
            if live and op < 0.25:
                m.end(live.pop(rng.randrange(len(live))))
            elif live and op < 0.35 and window == 0:
                r = rng.choice(live)
                m.rollback(r, rng.randint(0, m.seq_len[r]))
            elif live and op < 0.75:
                r = rng.choice(live)
                m.extend(r, rng.randint(1, 30))
                m.trim(r)
            else:
                m.begin(next_id)
                live.append(next_id)
                next_id += 1
                m.extend(live[-1], rng.randint(1, 60))
                m.trim(live[-1])
        except PoolExhausted:
            if next_id - 1 in m.seq_len and next_id - 1 not in live:
                m.end(next_id - 1)  # begun but no slot in the live list: cannot happen; keeps the test honest
        m.check()
        assert sorted(m.live) == sorted(live)
    # scattered pages: a fresh request lands on pages that are not one contiguous run
    for r in live[: len(live) // 2]:
        m.end(r)
        live.remove(r)
    if m.can_extend(None, 32) and m.slots.num_free:
        m.begin(10_000), m.extend(10_000, 32)
        t = m.table(0, 10_000)
        assert any(b != a + 1 for a, b in zip(t, t[1:])), t
    m.check()


def test_a_steps_description_is_packed_natively_and_reserves_all_or_nothing():
    """`pack_step`: pages for every entry or for none, and the layout that the kernels read (positions continue
    each request's sequence, a block table per group as wide as the longest one, sections on 16-byte bounds)."""
    import numpy as np

    m = CacheManager([(CacheNeed(2, 8, 0), None), (CacheNeed(1, 16, 0), None)], num_blocks=6, block_size=4, num_state_slots=3)
    m.begin(5), m.begin(9)
    m.extend(5, 6)
    buf = np.full(256, -7, dtype=np.int32)

    def pack(ids, q_lens, tokens, want=(), cap=256, limit=64):
        a = lambda x, t=np.int32: np.asarray(list(x), dtype=t)
        return m.pack_step(a(ids, np.int64), a(q_lens), a(tokens), a(want), a(()), a(()), a((11, 12, 13)), (2, 4), limit, buf, cap)

    offsets, widths, counts, total, max_q, max_kv = pack([5, 9], [1, 3], [40, 41, 42, 43], want=[0, 3])
    assert (max_q, max_kv, widths) == (3, 7, [2, 2]) and all(o % 4 == 0 for o in offsets) and total <= 256
    # one request decodes (row 0, 7 positions); the other's 3 tokens make two query tiles of 2 and one of 4
    assert counts == [1, 2, 1, 7, 1, 0]  # ... and one item in the decode work list, no request cut into parts
    sec = lambda i, n: buf[offsets[i]: offsets[i] + n].tolist()
    assert sec(0, 4) == [40, 41, 42, 43] and sec(1, 4) == [6, 0, 1, 2] and sec(2, 4) == [0, 1, 1, 1]
    assert sec(3, 3) == [0, 1, 4] and sec(4, 2) == [7, 3] and sec(5, 2) == [0, 1] and sec(6, 2) == [0, 3]
    assert sec(9, 1) == [0] and sec(10, 4) == [1, 2, 1, 0] and sec(11, 2) == [1, 0] and sec(12, 3) == [11, 12, 13]
    assert sec(13, 4) == [0, 0, 7, -1]  # (token row, request, keys it sees, whole)
    for gi in (0, 1):
        table = buf[offsets[14 + gi]: offsets[14 + gi] + 4].reshape(2, 2).tolist()
        assert table[0] == m.table(gi, 5) and table[1] == m.table(gi, 9) + [0]
    assert m.seq_len[5] == 7 and m.seq_len[9] == 3 and m.free_pages() == [3, 3]
    m.check()
    # the second entry does not fit: the first entry's reservation is undone as well
    with pytest.raises(PoolExhausted):
        pack([5, 9], [2, 14], list(range(16)))
    assert m.seq_len[5] == 7 and m.seq_len[9] == 3 and m.free_pages() == [3, 3]
    with pytest.raises(ValueError, match="limit is 8"):
        pack([5], [2], [1, 2], limit=8)
    with pytest.raises(BufferError) as e:
        pack([5], [1], [1], cap=8)
    assert e.value.args[0] > 8 and m.seq_len[5] == 7
    with pytest.raises(KeyError):
        pack([77], [1], [1])
    m.check()
    # the rows that decode are listed with the longest contexts first (the order in which the kernel's blocks are scheduled)
    big = CacheManager([(CacheNeed(2, 8, 0), None)], num_blocks=40, block_size=4, num_state_slots=5)
    for r, n in ((1, 5), (2, 40), (3, 12), (4, 40)):
        big.begin(r)
        big.extend(r, n)
    big.begin(8)
    a = lambda x, t=np.int32: np.asarray(list(x), dtype=t)
    offsets, _, counts, _, _, _ = big.pack_step(a([1, 2, 8, 3, 4], np.int64), a([1, 1, 3, 1, 1]), a(range(7)), a(()), a(()), a(()), a(()),
                                                (2, 4), 64, buf, 256)
    assert counts[0] == 4 and counts[3] == 41
    assert buf[offsets[9]: offsets[9] + 4].tolist() == [1, 6, 5, 0]  # requests 2 and 4 (41 keys, in their order), 3 (13), 1 (6)
    # contexts this short are never cut: the work list is the same rows, whole
    assert counts[4:] == [4, 0] and buf[offsets[13]: offsets[13] + 16].reshape(4, 4).tolist() == [
        [1, 1, 41, -1], [6, 4, 41, -1], [5, 3, 13, -1], [0, 0, 6, -1]]
    big.check()


def test_a_long_request_among_short_ones_comes_in_parts():
    """The decode work list: a context much longer than the mean is cut into parts of whole tiles of 64 keys, the
    longest items first, every key of every request exactly once, the parts' slots distinct; a bucket's list is
    padded with unused items and never has more extra items than it has room for."""
    import numpy as np

    lens = {1: 7900, 2: 200, 3: 150, 4: 5000, 5: 64, 6: 1}  # mean 2,219: parts of 2,240 keys; 7,900 makes three, 5,000 two
    m = CacheManager([(CacheNeed(2, 8, 0), None)], num_blocks=900, block_size=16, num_state_slots=8)
    for r, n in lens.items():
        m.begin(r)
        m.extend(r, n - 1)
    a = lambda x, t=np.int32: np.asarray(list(x), dtype=t)
    buf = np.zeros(8192, dtype=np.int32)

    def covered(items):
        """{row: None for a whole request, else its parts as (part, first key, end key, first slot, parts)}"""
        seen = {}
        slots = []
        for row, req, n, meta in items:
            if row < 0:
                assert req == -1 and meta == -1
                continue
            assert req == row and n == list(lens.values())[row]
            if meta < 0:
                assert row not in seen
                seen[row] = None
            else:
                first, c, parts = meta >> 8, (meta >> 4) & 15, meta & 15
                each = -(-(-(-n // parts)) // 64) * 64
                lo, hi = c * each, min(n, (c + 1) * each)
                assert 2 <= parts <= 15 and c < parts and lo < hi
                seen.setdefault(row, []).append((c, lo, hi, first, parts))
                slots.append(first + c)
        assert len(set(slots)) == len(slots) and sorted(slots) == list(range(len(slots)))
        return seen

    # an eager step: six decoding requests (rows 0..5)
    offsets, _, counts, _, _, _ = m.pack_step(a(lens, np.int64), a([1] * 6), a(range(6)), a(()), a(()), a(()), a(()), (2, 4), 8192, buf, 8192)
    n_items, n_slots = counts[4:]
    items = buf[offsets[13]: offsets[13] + 4 * n_items].reshape(n_items, 4).tolist()
    seen = covered(items)
    assert sorted(seen) == list(range(6))
    for row, n in enumerate(lens.values()):
        if seen[row] is None:
            assert n < 2 * 2240  # a whole request is shorter than two parts
            continue
        parts = sorted(seen[row])
        assert [p[0] for p in parts] == list(range(len(parts))) and parts[0][1] == 0 and parts[-1][2] == n
        assert all(x[2] == y[1] for x, y in zip(parts, parts[1:])) and len({(p[3], p[4]) for p in parts}) == 1
    assert len(seen[0]) == 3 and len(seen[3]) == 2 and n_slots == 5
    def keys_of(row, n, meta):
        if meta < 0:
            return n
        c, parts = (meta >> 4) & 15, meta & 15
        each = -(-(-(-n // parts)) // 64) * 64
        return min(n, (c + 1) * each) - c * each

    sizes = [keys_of(row, n, meta) for row, _, n, meta in items]
    assert sizes == sorted(sizes, reverse=True)
    for r in lens:
        m.rollback(r, lens[r] - 1)
    # a graph bucket of 8 rows with room for 3 extra items: the parts grow until they fit
    off = {"positions": 0, "token_req": 8, "kv_len": 16, "slots": 24, "work": 32}
    table_off = (__import__("ctypes").c_int * 1)(128)
    m.pack_decode(a(lens, np.int64), 8, 8192, buf, off, table_off, 512, n_work=9)
    items = buf[32: 32 + 36].reshape(9, 4).tolist()
    seen = covered(items)
    assert sorted(seen) == list(range(6)) and sum(1 for it in items if it[0] < 0) == 0
    assert sum(len(v) - 1 for v in seen.values() if v) == 3
    # room for two: parts twice as long, and neither request is twice as long as those
    for r in lens:
        m.rollback(r, lens[r] - 1)
    m.pack_decode(a(lens, np.int64), 8, 8192, buf, off, table_off, 512, n_work=8)
    items = buf[32: 32 + 32].reshape(8, 4).tolist()
    assert all(v is None for v in covered(items).values()) and sum(1 for it in items if it[0] < 0) == 2
    m.check()


def test_a_decode_steps_description_for_a_graph_bucket():
    import ctypes

    import numpy as np

    m = manager(num_blocks=8, block_size=4, lanes=1, slots=3)
    m.begin(3), m.begin(4)
    m.extend(3, 4), m.extend(4, 2)
    buf = np.full(64, -7, dtype=np.int32)
    off = {"positions": 0, "token_req": 4, "kv_len": 8, "slots": 12}
    m.pack_decode(np.asarray([4, 3], dtype=np.int64), 4, 64, buf, off, (ctypes.c_int * 1)(16), 5)
    assert buf[0:4].tolist() == [2, 4, 0, 0] and buf[4:8].tolist() == [0, 1, -1, -1]       # padding rows: request -1
    assert buf[8:12].tolist() == [3, 5, 0, 0] and buf[12:16].tolist() == [1, 0, 3, 3]        # ... and the scratch slot
    assert buf[16:17].tolist() == m.table(0, 4) and buf[21:23].tolist() == m.table(0, 3)    # request 3 took a second page
    assert m.seq_len[3] == 5 and m.seq_len[4] == 3
    with pytest.raises(ValueError, match="wider"):
        m.pack_decode(np.asarray([3], dtype=np.int64), 4, 64, buf, off, (ctypes.c_int * 1)(16), 1)
    m.check()
