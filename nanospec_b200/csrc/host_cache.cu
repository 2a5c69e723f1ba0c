// The cache manager and the step description, host side (no device code in this file).
//
// Which pages and which state slot every live request holds, for all cache groups of a model, and the
// packing of one step's description (token ids, positions, request of each token, lengths, state slots,
// wanted rows, one block table per group) into one pinned buffer that is copied to the device once.
// Behaviour follows the reference's allocator (kv/allocator.py:22-85: a LIFO free list that hands out page 0
// first and reuses the page freed last, a block table per request, exhaustion reported before anything is
// changed, every page in exactly one place) and its batch description (kv/cache.py:113-157), with what this
// engine adds: several groups with pools of their own, windows that give pages back while a request runs,
// and slots of fixed-size state.  The Python class nanospec_b200.cache.CacheManager is a thin face of this.
#include <algorithm>
#include <cstring>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace {

enum : int { NS_ERR_EXHAUSTED = 4, NS_ERR_NOT_LIVE = 5, NS_ERR_SMALL = 6, NS_ERR_INVARIANT = 7 };
constexpr int kReleased = -1;  // block-table entry of a page that a window has passed

struct Group {
    int page_size = 0, window = 0, num_pages = 0;
    std::vector<int> free_list;  // back() goes out next
    std::vector<unsigned char> is_free;

    long long blocks_for(long long len) const { return (len + page_size - 1) / page_size; }
    // first logical block that a query at position >= len can still read
    long long first_needed_block(long long len) const {
        if (window <= 0) return 0;
        const long long first_pos = len - window + 1;
        return (first_pos > 0 ? first_pos : 0) / page_size;
    }
};

struct Table {
    std::vector<int> pages;  // one entry per logical block, kReleased once given back
    int first_live = 0;
};

struct Request {
    long long seq_len = 0;
    int slot = -1;
    std::vector<Table> tables;  // one per group
};

struct Cache {
    std::vector<Group> groups;
    std::unordered_map<long long, Request> live;
    std::vector<long long> order;  // live request ids in the order of their begin()
    std::vector<int> free_slots;   // back() goes out next
    int num_slots = 0;
    std::vector<int> fresh;        // slots handed out since the last step: their state must be zeroed
};

Cache* as_cache(void* h) { return static_cast<Cache*>(h); }

int give_page(Group& g, int p) {
    if (p < 0 || p >= g.num_pages || g.is_free[p]) NS_FAIL(NS_ERR_INVARIANT, "page %d freed twice or never handed out", p);
    g.is_free[p] = 1;
    g.free_list.push_back(p);
    return NS_OK;
}

// pages every group must take so that `r` (nullptr: a new request) reaches new_len
void need_of(const Cache& c, const Request* r, long long new_len, int* out) {
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        const long long have = r ? (long long)r->tables[gi].pages.size() : 0;
        const long long n = c.groups[gi].blocks_for(new_len) - have;
        out[gi] = (int)(n > 0 ? n : 0);
    }
}

int extend_request(Cache& c, long long id, Request& r, long long n_tokens) {
    const long long new_len = r.seq_len + n_tokens;
    int need[16];
    need_of(c, &r, new_len, need);
    for (size_t gi = 0; gi < c.groups.size(); ++gi)
        if (need[gi] > (int)c.groups[gi].free_list.size())
            NS_FAIL(NS_ERR_EXHAUSTED, "request %lld needs %d pages, %d free", id, need[gi], (int)c.groups[gi].free_list.size());
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        Group& g = c.groups[gi];
        for (int i = 0; i < need[gi]; ++i) {
            const int p = g.free_list.back();
            g.free_list.pop_back();
            g.is_free[p] = 0;
            r.tables[gi].pages.push_back(p);
        }
    }
    r.seq_len = new_len;
    return NS_OK;
}

int rollback_request(Cache& c, Request& r, long long seq_len) {
    if (seq_len < 0 || seq_len > r.seq_len) NS_FAIL(NS_ERR_INVARIANT, "rollback goes backwards only");
    for (size_t gi = 0; gi < c.groups.size(); ++gi)
        if (c.groups[gi].blocks_for(seq_len) < r.tables[gi].first_live)
            NS_FAIL(NS_ERR_INVARIANT, "cannot roll back behind pages that a window has already released");
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        Table& t = r.tables[gi];
        const size_t keep = (size_t)c.groups[gi].blocks_for(seq_len);
        for (size_t i = keep; i < t.pages.size(); ++i) {
            const int st = give_page(c.groups[gi], t.pages[i]);
            if (st != NS_OK) return st;
        }
        if (t.pages.size() > keep) t.pages.resize(keep);
    }
    r.seq_len = seq_len;
    return NS_OK;
}

int trim_request(Cache& c, Request& r, int* released) {
    for (size_t gi = 0; gi < c.groups.size(); ++gi) {
        Group& g = c.groups[gi];
        Table& t = r.tables[gi];
        const int first = (int)std::min<long long>(g.first_needed_block(r.seq_len), (long long)t.pages.size());
        for (int i = t.first_live; i < first; ++i) {
            const int st = give_page(g, t.pages[i]);
            if (st != NS_OK) return st;
            t.pages[i] = kReleased;
            ++*released;
        }
        if (first > t.first_live) t.first_live = first;
    }
    return NS_OK;
}

inline int pad4(long long n) { return (int)((n + 3) & ~3ll); }

}  // namespace

#define NS_FIND(c, id, r)                                                            \
    auto it_ = (c)->live.find(id);                                                   \
    if (it_ == (c)->live.end()) NS_FAIL(NS_ERR_NOT_LIVE, "request %lld is not live", (long long)(id)); \
    Request& r = it_->second

NS_API int ns_cache_create(int n_groups, const int* page_size, const int* window, int num_pages, int num_slots, void** out) {
    if (n_groups < 0 || n_groups > 16) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_cache_create: %d cache groups (at most 16)", n_groups);
    if (num_pages <= 0 || num_slots <= 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_cache_create: a pool needs at least one page and one slot");
    Cache* c = new Cache();
    c->groups.resize(n_groups);
    for (int gi = 0; gi < n_groups; ++gi) {
        Group& g = c->groups[gi];
        if (page_size[gi] <= 0) { delete c; NS_FAIL(NS_ERR_ARGUMENT, "ns_cache_create: page size %d", page_size[gi]); }
        g.page_size = page_size[gi];
        g.window = window[gi];
        g.num_pages = num_pages;
        g.free_list.resize(num_pages);
        for (int p = 0; p < num_pages; ++p) g.free_list[p] = num_pages - 1 - p;  // page 0 goes out first
        g.is_free.assign(num_pages, 1);
    }
    c->num_slots = num_slots;
    c->free_slots.resize(num_slots);
    for (int s = 0; s < num_slots; ++s) c->free_slots[s] = num_slots - 1 - s;    // slot 0 goes out first
    *out = c;
    return NS_OK;
}

NS_API int ns_cache_destroy(void* h) {
    delete as_cache(h);
    return NS_OK;
}

NS_API int ns_cache_begin(void* h, long long id) {
    Cache* c = as_cache(h);
    if (c->live.count(id)) NS_FAIL(NS_ERR_INVARIANT, "request %lld is already live", id);
    if (c->free_slots.empty()) NS_FAIL(NS_ERR_EXHAUSTED, "no free state slot");  // before anything else changes
    Request r;
    r.slot = c->free_slots.back();
    c->free_slots.pop_back();
    r.tables.resize(c->groups.size());
    c->fresh.push_back(r.slot);
    c->live.emplace(id, std::move(r));
    c->order.push_back(id);
    return NS_OK;
}

// Room for n_tokens more positions in every group, or NS_ERR_EXHAUSTED with everything as it was.
NS_API int ns_cache_extend(void* h, long long id, long long n_tokens) {
    Cache* c = as_cache(h);
    NS_FIND(c, id, r);
    if (n_tokens < 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_cache_extend: %lld tokens", n_tokens);
    return extend_request(*c, id, r, n_tokens);
}

// After a step: the pages that no later query of the request can read (wholly behind a window) go back.
NS_API int ns_cache_trim(void* h, long long id, int* released) {
    Cache* c = as_cache(h);
    NS_FIND(c, id, r);
    *released = 0;
    return trim_request(*c, r, released);
}

NS_API int ns_cache_trim_many(void* h, int n, const long long* ids) {
    Cache* c = as_cache(h);
    int released = 0;
    for (int i = 0; i < n; ++i) {
        NS_FIND(c, ids[i], r);
        const int st = trim_request(*c, r, &released);
        if (st != NS_OK) return st;
    }
    return NS_OK;
}

NS_API int ns_cache_rollback(void* h, long long id, long long seq_len) {
    Cache* c = as_cache(h);
    NS_FIND(c, id, r);
    return rollback_request(*c, r, seq_len);
}

NS_API int ns_cache_end(void* h, long long id) {
    Cache* c = as_cache(h);
    NS_FIND(c, id, r);
    for (size_t gi = 0; gi < c->groups.size(); ++gi)
        for (int p : r.tables[gi].pages)
            if (p != kReleased) {
                const int st = give_page(c->groups[gi], p);
                if (st != NS_OK) return st;
            }
    c->free_slots.push_back(r.slot);
    c->live.erase(it_);
    c->order.erase(std::find(c->order.begin(), c->order.end(), id));
    return NS_OK;
}

// id < 0: a request that is not live yet
NS_API int ns_cache_need(void* h, long long id, long long new_len, int* out) {
    Cache* c = as_cache(h);
    const Request* r = nullptr;
    if (id >= 0) {
        auto it = c->live.find(id);
        if (it != c->live.end()) r = &it->second;
    }
    need_of(*c, r, new_len, out);
    return NS_OK;
}

NS_API int ns_cache_free_pages(void* h, int* out) {
    Cache* c = as_cache(h);
    for (size_t gi = 0; gi < c->groups.size(); ++gi) out[gi] = (int)c->groups[gi].free_list.size();
    return NS_OK;
}

NS_API int ns_cache_held_pages(void* h, long long id, int* out) {
    Cache* c = as_cache(h);
    NS_FIND(c, id, r);
    for (size_t gi = 0; gi < c->groups.size(); ++gi) out[gi] = (int)r.tables[gi].pages.size() - r.tables[gi].first_live;
    return NS_OK;
}

// seq_len and slot of a request; *seq_len = -1 when it is not live (no error)
NS_API int ns_cache_lookup(void* h, long long id, long long* seq_len, int* slot) {
    Cache* c = as_cache(h);
    auto it = c->live.find(id);
    *seq_len = it == c->live.end() ? -1 : it->second.seq_len;
    *slot = it == c->live.end() ? -1 : it->second.slot;
    return NS_OK;
}

NS_API int ns_cache_counts(void* h, int* n_live, int* free_slots, int* n_fresh) {
    Cache* c = as_cache(h);
    *n_live = (int)c->live.size();
    *free_slots = (int)c->free_slots.size();
    *n_fresh = (int)c->fresh.size();
    return NS_OK;
}

NS_API int ns_cache_live(void* h, long long* out, int cap) {
    Cache* c = as_cache(h);
    if ((int)c->order.size() > cap) NS_FAIL(NS_ERR_SMALL, "ns_cache_live: %d live requests", (int)c->order.size());
    std::copy(c->order.begin(), c->order.end(), out);
    return NS_OK;
}

NS_API int ns_cache_table(void* h, int group, long long id, int* out, int cap, int* n, int* first_live) {
    Cache* c = as_cache(h);
    NS_FIND(c, id, r);
    if (group < 0 || group >= (int)c->groups.size()) NS_FAIL(NS_ERR_ARGUMENT, "ns_cache_table: group %d", group);
    const Table& t = r.tables[group];
    *n = (int)t.pages.size();
    *first_live = t.first_live;
    if (*n > cap) NS_FAIL(NS_ERR_SMALL, "ns_cache_table: %d entries", *n);
    std::copy(t.pages.begin(), t.pages.end(), out);
    return NS_OK;
}

NS_API int ns_cache_free_list(void* h, int group, int* out, int cap) {
    Cache* c = as_cache(h);
    const Group& g = c->groups[group];
    if ((int)g.free_list.size() > cap) NS_FAIL(NS_ERR_SMALL, "ns_cache_free_list: %d free pages", (int)g.free_list.size());
    std::copy(g.free_list.begin(), g.free_list.end(), out);
    return NS_OK;
}

NS_API int ns_cache_take_fresh(void* h, int* out, int cap) {
    Cache* c = as_cache(h);
    if ((int)c->fresh.size() > cap) NS_FAIL(NS_ERR_SMALL, "ns_cache_take_fresh: %d slots", (int)c->fresh.size());
    std::copy(c->fresh.begin(), c->fresh.end(), out);
    c->fresh.clear();
    return NS_OK;
}

// No page lost, held twice or freed twice; tables as long as their sequences need; every slot in one place.
NS_API int ns_cache_check(void* h) {
    Cache* c = as_cache(h);
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        const Group& g = c->groups[gi];
        std::vector<int> seen(g.num_pages, 0);
        for (int p : g.free_list) {
            if (p < 0 || p >= g.num_pages || !g.is_free[p]) NS_FAIL(NS_ERR_INVARIANT, "group %d: free list holds page %d wrongly", (int)gi, p);
            ++seen[p];
        }
        for (const auto& kv : c->live) {
            const Table& t = kv.second.tables[gi];
            if ((long long)t.pages.size() != g.blocks_for(kv.second.seq_len))
                NS_FAIL(NS_ERR_INVARIANT, "group %d: request %lld has %d table entries for %lld positions", (int)gi, kv.first,
                        (int)t.pages.size(), kv.second.seq_len);
            for (int i = 0; i < (int)t.pages.size(); ++i) {
                const int p = t.pages[i];
                if (i < t.first_live) {
                    if (p != kReleased) NS_FAIL(NS_ERR_INVARIANT, "group %d: request %lld keeps a page behind its window", (int)gi, kv.first);
                    continue;
                }
                if (p < 0 || p >= g.num_pages || g.is_free[p]) NS_FAIL(NS_ERR_INVARIANT, "group %d: request %lld holds page %d wrongly", (int)gi, kv.first, p);
                ++seen[p];
            }
        }
        for (int p = 0; p < g.num_pages; ++p)
            if (seen[p] != 1) NS_FAIL(NS_ERR_INVARIANT, "group %d: page %d is %s", (int)gi, p, seen[p] ? "held twice" : "lost");
    }
    std::vector<int> slot_seen(c->num_slots, 0);
    for (int s : c->free_slots) ++slot_seen[s];
    for (const auto& kv : c->live) ++slot_seen[kv.second.slot];
    for (int s = 0; s < c->num_slots; ++s)
        if (slot_seen[s] != 1) NS_FAIL(NS_ERR_INVARIANT, "state slot %d is %s", s, slot_seen[s] ? "held twice" : "lost");
    if (c->order.size() != c->live.size()) NS_FAIL(NS_ERR_INVARIANT, "the list of live requests is out of step");
    return NS_OK;
}

// ---------------------------------------------------------------------------------------------------
// The decode attention kernel's work list.  Its blocks are per request, so a request whose context is much longer
// than the others' would stream alone long after they are done.  A request of at least twice the mean context is cut
// into parts of about the mean (at least 512 keys, whole tiles of 64, at most 15 parts, and no more extra items than
// `extra_cap`: the parts grow until they fit); each part is an item of its own, and the kernel adds the parts up.  Items are
// (token row, request, keys the request sees, meta): meta = -1 for a whole request, else first slot << 8 | part << 4 |
// parts, where part c of a request of `len` keys is the keys [c * each, min(len, (c + 1) * each)) with each =
// ceil(len / parts) rounded up to whole tiles, and the request's parts take the slots first .. first + parts - 1
// of the kernel's scratch.  The longest items come first: blocks are scheduled in that order.  `rows[i]` is the
// token row of entry i, `reqs[i]` its row of the block tables, `lens[i]` the keys it sees.
// ---------------------------------------------------------------------------------------------------
struct WorkItem { int row, req, len, meta; };

static std::vector<WorkItem> plan_decode_work(const std::vector<int>& rows, const std::vector<int>& req_rows,
                                              const std::vector<long long>& lens, long long extra_cap, int* n_slots) {
    const int n = (int)rows.size();
    std::vector<WorkItem> items;
    *n_slots = 0;
    if (n == 0) return items;
    long long total = 0;
    for (long long v : lens) total += v;
    long long part = std::max(512ll, ((total / n + 63) / 64) * 64);
    // a request is cut only when it is at least twice as long as a part
    auto parts_of = [&](long long len) { return (int)std::min(15ll, std::max(1ll, len / part)); };
    for (;;) {
        long long extra = 0;
        for (long long v : lens) extra += parts_of(v) - 1;
        if (extra <= extra_cap) break;
        part *= 2;
    }
    struct Keyed { WorkItem item; long long keys; };
    std::vector<Keyed> keyed;
    keyed.reserve(n + (size_t)extra_cap);
    for (int i = 0; i < n; ++i) {
        int parts = std::max(1, parts_of(lens[i]));
        // whole tiles: rounding a part up may leave the last parts empty; fewer parts then
        while (parts > 1 && (long long)(parts - 1) * ((((lens[i] + parts - 1) / parts + 63) / 64) * 64) >= lens[i]) --parts;
        if (parts == 1) {
            keyed.push_back({{rows[i], req_rows[i], (int)lens[i], -1}, lens[i]});
            continue;
        }
        const long long each = (((lens[i] + parts - 1) / parts + 63) / 64) * 64;
        for (int c = 0; c < parts; ++c) {
            const long long from = c * each, to = std::min(lens[i], from + each);
            keyed.push_back({{rows[i], req_rows[i], (int)lens[i], (*n_slots << 8) | (c << 4) | parts}, to - from});
        }
        *n_slots += parts;
    }
    std::stable_sort(keyed.begin(), keyed.end(), [](const Keyed& x, const Keyed& y) { return x.keys > y.keys; });
    items.reserve(keyed.size());
    for (const Keyed& k : keyed) items.push_back(k.item);
    return items;
}

// ---------------------------------------------------------------------------------------------------
// One step's description.  Reserves pages for every entry (all of them, or none: NS_ERR_EXHAUSTED and
// NS_ERR_ARGUMENT leave the cache as it was) and lays out, in `buf` (int32, 16-byte aligned sections):
//   0 token ids [N]   1 positions [N]   2 request of each token [N]   3 qo_indptr [B+1]   4 kv_len [B]
//   5 state slots [B] 6 wanted rows [n_want]   7 take_dst [n_take]   8 take_src [n_take]
//   9 the token rows of the requests that bring one token [counts[0]]
//   10, 11 the query tiles of the requests that bring more, as (request, offset among its tokens) pairs, for tiles
//      of tile_q[0] and of tile_q[1] queries [2 * counts[1]], [2 * counts[2]]; the tiles that see the most keys first
//   12 whatever the caller wants copied along [n_extra] (the sampling options of the step's sampled rows)
//   13 the decode attention kernel's work list [4 * counts[4]] (see plan_decode_work; counts[5] slots of scratch)
//   14.. one block table per group, [B, width] with width = the longest table among the entries (>= 1)
// offsets[14 + groups], widths[groups]; counts[3] = the longest sequence among the one-token requests (0: none);
// *total = ints used.  NS_ERR_SMALL (nothing changed) when cap is too small, with *total = what is needed.
// ---------------------------------------------------------------------------------------------------
NS_API int ns_step_pack(void* h, int B, const long long* ids, const int* q_lens, const int* tokens, int n_want,
                        const int* want_rows, int n_take, const int* take_dst, const int* take_src, int n_extra,
                        const int* extra, const int* tile_q, long long max_positions, int* buf, long long cap, int* offsets,
                        int* widths, long long* counts, long long* total, int* max_q, long long* max_kv) {
    Cache* c = as_cache(h);
    const int G = (int)c->groups.size();
    std::vector<Request*> reqs(B);
    long long N = 0, n_decode = 0, n_tiles[2] = {0, 0}, max_kv_decode = 0;
    *max_q = 0;
    *max_kv = 0;
    std::vector<long long> table_len(G, 1);
    for (int b = 0; b < B; ++b) {
        auto it = c->live.find(ids[b]);
        if (it == c->live.end()) NS_FAIL(NS_ERR_NOT_LIVE, "request %lld is not live", ids[b]);
        reqs[b] = &it->second;
        if (q_lens[b] <= 0) NS_FAIL(NS_ERR_ARGUMENT, "request %lld brings no tokens to the step", ids[b]);
        const long long end = reqs[b]->seq_len + q_lens[b];
        if (end > max_positions)
            NS_FAIL(NS_ERR_ARGUMENT, "request %lld would reach %lld positions; the model's limit is %lld", ids[b], end, max_positions);
        N += q_lens[b];
        *max_q = std::max(*max_q, q_lens[b]);
        *max_kv = std::max(*max_kv, end);
        if (q_lens[b] == 1) {
            ++n_decode;
            max_kv_decode = std::max(max_kv_decode, end);
        } else {
            for (int t = 0; t < 2; ++t) n_tiles[t] += (q_lens[b] + tile_q[t] - 1) / tile_q[t];
        }
        for (int gi = 0; gi < G; ++gi) table_len[gi] = std::max(table_len[gi], c->groups[gi].blocks_for(end));
    }
    // the work list of the requests that bring one token (their token rows are known already: rows run in entry order)
    std::vector<int> work_rows, work_reqs;
    std::vector<long long> work_lens;
    {
        long long row = 0;
        for (int b = 0; b < B; ++b) {
            if (q_lens[b] == 1) {
                work_rows.push_back((int)row);
                work_reqs.push_back(b);
                work_lens.push_back(reqs[b]->seq_len + 1);
            }
            row += q_lens[b];
        }
    }
    int n_slots = 0;
    const std::vector<WorkItem> work = plan_decode_work(work_rows, work_reqs, work_lens, n_decode, &n_slots);
    long long at = 0;
    const long long sizes[14] = {N, N, N, (long long)B + 1, B, B, n_want, n_take, n_take, n_decode, 2 * n_tiles[0], 2 * n_tiles[1],
                                 n_extra, 4 * (long long)work.size()};
    for (int s = 0; s < 14; ++s) { offsets[s] = (int)at; at += pad4(sizes[s]); }
    for (int gi = 0; gi < G; ++gi) {
        widths[gi] = (int)table_len[gi];
        offsets[14 + gi] = (int)at;
        at += pad4((long long)B * table_len[gi]);
    }
    *total = at;
    counts[0] = n_decode, counts[1] = n_tiles[0], counts[2] = n_tiles[1], counts[3] = max_kv_decode;
    counts[4] = (long long)work.size(), counts[5] = n_slots;
    if (at > cap) NS_FAIL(NS_ERR_SMALL, "ns_step_pack: the description needs %lld ints, the buffer holds %lld", at, cap);
    // reserve: everything or nothing
    std::vector<long long> before(B);
    for (int b = 0; b < B; ++b) {
        before[b] = reqs[b]->seq_len;
        const int st = extend_request(*c, ids[b], *reqs[b], q_lens[b]);
        if (st != NS_OK) {
            char keep[sizeof(ns_error_text)];
            memcpy(keep, ns_error_text, sizeof(keep));
            for (int u = b - 1; u >= 0; --u) rollback_request(*c, *reqs[u], before[u]);
            memcpy(ns_error_text, keep, sizeof(keep));
            return st;
        }
    }
    memcpy(buf + offsets[0], tokens, sizeof(int) * N);
    int* positions = buf + offsets[1];
    int* token_req = buf + offsets[2];
    int* qo = buf + offsets[3];
    int* kv_len = buf + offsets[4];
    int* slots = buf + offsets[5];
    int* decode_rows = buf + offsets[9];
    long long row = 0, d = 0;
    qo[0] = 0;
    for (int b = 0; b < B; ++b) {
        for (int i = 0; i < q_lens[b]; ++i) {
            positions[row + i] = (int)(before[b] + i);
            token_req[row + i] = b;
        }
        if (q_lens[b] == 1) decode_rows[d++] = (int)row;
        row += q_lens[b];
        qo[b + 1] = (int)row;
        kv_len[b] = (int)reqs[b]->seq_len;
        slots[b] = reqs[b]->slot;
    }
    // the decode attention kernel's blocks are scheduled in this order: the requests with the most keys first, so that
    // no long one starts when the others are done
    std::stable_sort(decode_rows, decode_rows + d, [&](int x, int y) { return kv_len[token_req[x]] > kv_len[token_req[y]]; });
    if (n_want) memcpy(buf + offsets[6], want_rows, sizeof(int) * n_want);
    if (n_take) {
        memcpy(buf + offsets[7], take_dst, sizeof(int) * n_take);
        memcpy(buf + offsets[8], take_src, sizeof(int) * n_take);
    }
    if (n_extra) memcpy(buf + offsets[12], extra, sizeof(int) * n_extra);
    if (!work.empty()) memcpy(buf + offsets[13], work.data(), sizeof(WorkItem) * work.size());
    // query tiles of the prompt portions; blocks are scheduled in this order, so the tiles that see the most keys
    // (the last ones of the longest sequences) come first
    struct Tile { int req, off; long long keys; };
    for (int t = 0; t < 2; ++t) {
        std::vector<Tile> tiles;
        tiles.reserve(n_tiles[t]);
        for (int b = 0; b < B; ++b) {
            if (q_lens[b] == 1) continue;
            for (int off = 0; off < q_lens[b]; off += tile_q[t])
                tiles.push_back({b, off, before[b] + std::min(off + tile_q[t], q_lens[b])});
        }
        std::stable_sort(tiles.begin(), tiles.end(), [](const Tile& x, const Tile& y) { return x.keys > y.keys; });
        int* out = buf + offsets[10 + t];
        for (size_t i = 0; i < tiles.size(); ++i) { out[2 * i] = tiles[i].req; out[2 * i + 1] = tiles[i].off; }
    }
    for (int gi = 0; gi < G; ++gi) {
        int* table = buf + offsets[14 + gi];
        const int W = widths[gi];
        for (int b = 0; b < B; ++b) {
            const std::vector<int>& pages = reqs[b]->tables[gi].pages;
            std::copy(pages.begin(), pages.end(), table + (long long)b * W);
            std::fill(table + (long long)b * W + pages.size(), table + (long long)(b + 1) * W, 0);
        }
    }
    return NS_OK;
}

// The description of a decode-only step of a captured graph's bucket: `size` rows of which the first B are
// requests with one token each, the rest padding (request -1, length 0, the scratch state slot).  Reserves
// one position per request (all or none) and writes positions, token_req, kv_len, slots and, for every group,
// the block table rows of width `width` into `buf` at the given offsets; with n_work > 0 also the decode attention
// kernel's work list of exactly n_work items (16-byte aligned at off_work; at most n_work - B extra parts).
NS_API int ns_step_pack_decode(void* h, int B, int size, const long long* ids, long long max_positions, int scratch_slot,
                               int* buf, int off_positions, int off_token_req, int off_kv_len, int off_slots,
                               const int* table_off, int width, int off_work, int n_work) {
    Cache* c = as_cache(h);
    const int G = (int)c->groups.size();
    if (B > size) NS_FAIL(NS_ERR_ARGUMENT, "ns_step_pack_decode: %d requests in a bucket of %d", B, size);
    std::vector<Request*> reqs(B);
    for (int b = 0; b < B; ++b) {
        auto it = c->live.find(ids[b]);
        if (it == c->live.end()) NS_FAIL(NS_ERR_NOT_LIVE, "request %lld is not live", ids[b]);
        reqs[b] = &it->second;
        if (reqs[b]->seq_len + 1 > max_positions)
            NS_FAIL(NS_ERR_ARGUMENT, "request %lld would reach %lld positions; the model's limit is %lld", ids[b],
                    reqs[b]->seq_len + 1, max_positions);
        for (int gi = 0; gi < G; ++gi)
            if (c->groups[gi].blocks_for(reqs[b]->seq_len + 1) > width)
                NS_FAIL(NS_ERR_ARGUMENT, "request %lld needs a block table wider than the graph's %d", ids[b], width);
    }
    for (int b = 0; b < B; ++b) {
        const int st = extend_request(*c, ids[b], *reqs[b], 1);
        if (st != NS_OK) {
            char keep[sizeof(ns_error_text)];
            memcpy(keep, ns_error_text, sizeof(keep));
            for (int u = b - 1; u >= 0; --u) rollback_request(*c, *reqs[u], reqs[u]->seq_len - 1);
            memcpy(ns_error_text, keep, sizeof(keep));
            return st;
        }
    }
    for (int b = 0; b < size; ++b) {
        const bool real = b < B;
        buf[off_positions + b] = real ? (int)(reqs[b]->seq_len - 1) : 0;
        buf[off_token_req + b] = real ? b : -1;
        buf[off_kv_len + b] = real ? (int)reqs[b]->seq_len : 0;
        buf[off_slots + b] = real ? reqs[b]->slot : scratch_slot;
    }
    if (n_work > 0) {
        // the work list of the bucket: n_work items, the unused ones with row -1
        if (n_work < B) NS_FAIL(NS_ERR_ARGUMENT, "ns_step_pack_decode: a work list of %d items for %d requests", n_work, B);
        std::vector<int> rows(B);
        std::vector<long long> lens(B);
        for (int b = 0; b < B; ++b) { rows[b] = b; lens[b] = reqs[b]->seq_len; }
        int n_slots = 0;
        const std::vector<WorkItem> work = plan_decode_work(rows, rows, lens, n_work - B, &n_slots);
        WorkItem* out = reinterpret_cast<WorkItem*>(buf + off_work);
        for (int i = 0; i < n_work; ++i) out[i] = i < (int)work.size() ? work[i] : WorkItem{-1, -1, 0, -1};
    }
    for (int gi = 0; gi < G; ++gi)
        for (int b = 0; b < B; ++b) {
            const std::vector<int>& pages = reqs[b]->tables[gi].pages;
            // entries behind a window are never read; the row is written from its first live entry on
            const int first = reqs[b]->tables[gi].first_live;
            std::copy(pages.begin() + first, pages.end(), buf + table_off[gi] + (long long)b * width + first);
        }
    return NS_OK;
}
