// Pieces shared by the bfloat16 attention kernels: tile sizes and the loader that brings 64
// keys and values of one kv head from scattered cache pages into padded shared-memory tiles.
#pragma once

#include "mma_utils.cuh"

namespace {

constexpr int kTileKeys = 64;
constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

// Rows key0 .. key0+63 of one kv head: cache[page, hk, offset, :] with page = bt[key / page_size].
// Rows before key_lo (their pages may already have been given back behind a window) and rows at or
// beyond key_end are not read but zero-filled (a masked weight of zero must not meet a NaN).
template <int D, int THREADS = kThreads>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* ks, __nv_bfloat16* vs, const __nv_bfloat16* k_cache,
                                             const __nv_bfloat16* v_cache, const int* bt, int key0, int key_lo, int key_end,
                                             int hk, int nkv, int page_size, int page_shift) {
    constexpr int kChunks = D / 8;
    constexpr int kItems = (kTileKeys * kChunks + THREADS - 1) / THREADS;  // 16-byte pieces per thread and tensor
    // When the threads divide evenly over the pieces of a row, a thread keeps the same piece of
    // the row for every item and its rows advance by a constant: no division per item.
    constexpr bool kRegular = THREADS % kChunks == 0;
    constexpr int kRowStep = kRegular ? THREADS / kChunks : 0;
    const int ch0 = kRegular ? threadIdx.x % kChunks : 0;
    const int row0 = kRegular ? threadIdx.x / kChunks : 0;
    // first the block-table entries of all of this thread's rows (independent loads), then the copies:
    // the copies are ordered against other memory operations, and a table lookup between two of them
    // would cost a full load latency each time
    int page[kItems];
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const int c = threadIdx.x + i * THREADS;
        const int row = kRegular ? row0 + i * kRowStep : c / kChunks;
        const int key = key0 + row;
        const bool valid = c < kTileKeys * kChunks && key >= key_lo && key < key_end;
        // page_shift >= 0: the page size is a power of two (no integer division per row)
        page[i] = valid ? __ldg(bt + (page_shift >= 0 ? key >> page_shift : key / page_size)) : -1;
    }
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
        const int c = threadIdx.x + i * THREADS;
        if (c >= kTileKeys * kChunks) break;
        const int row = kRegular ? row0 + i * kRowStep : c / kChunks;
        const int ch = kRegular ? ch0 : c - row * kChunks;
        const int key = key0 + row;
        const bool valid = page[i] >= 0;
        size_t off = 0;
        if (valid) {
            const int within = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
            off = (((size_t)page[i] * nkv + hk) * page_size + within) * D + ch * 8;
        }
        ns_cp_async16(NsTile<D>::at(ks, row, ch * 8), k_cache + off, valid);
        ns_cp_async16(NsTile<D>::at(vs, row, ch * 8), v_cache + off, valid);
    }
}

}  // namespace
