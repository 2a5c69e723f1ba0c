// Prefill attention on the 5th-generation tensor cores (head sizes 64 and 128, bfloat16): portions of
// prompts, causal by absolute position, keys and values read from the paged cache.
//
// One block = 256 consecutive query tokens of one request (two tiles of 128, each with its own softmax
// warpgroup and accumulator; they share every block of keys) and one query head.  Per 64 keys and tile:
//   S = Q K^T        tcgen05.mma, Q and K tiles in 128-byte-swizzled shared memory (TMA), S in TMEM
//   softmax          128 threads, one query row each (the row of S is read with tcgen05.ld, so the
//                    running maximum and sum need no exchange between threads), fp32, base 2;
//                    the weights go back to TMEM as bf16 pairs over the first half of the scores
//                    they came from; the accumulator O in TMEM is rescaled only when some row's
//                    maximum has grown by more than a factor 256
//   O += P V         tcgen05.mma, P read from TMEM (so the tensor core's shared-memory reads are V
//                    alone), V as it lies in the cache (dim contiguous: an MN-major operand)
// Warp roles: warp 0 (one elected lane) issues the TMA loads - the keys of a block come from 64/page_size
// cache pages, found through the request's block table; warp 1 issues the MMAs of S = Q K^T and owns the
// TMEM allocation; warp 2 issues the MMAs of O += P V; warps 3-6 and 7-10 are the softmax threads of the
// two tiles and write the output.  S is double buffered in TMEM, so the scores of blocks j+1 and j+2 are
// computed while block j is in the softmax; the scores of block j+2 go where P of block j lies, once the
// product that read it has completed (an mbarrier that the P V issuer commits to).  The two products have
// a warp each because issuing a tcgen05.mma blocks until the tensor core takes it: one warp that also
// waited for the softmax left the tensor core idle during its waits.
//
// Every mbarrier wait is bounded (two seconds); a wait that runs out sets *error_flag and the
// block winds down.  Other head sizes, page sizes other than 8/16/32/64 and windows
// are served by the m16n8k16 kernel of attention_prefill.cu.  A second kernel below takes heads of 64 in groups
// of an even size, two query heads to a block.
#include "tcgen05_utils.cuh"

namespace {

constexpr int kBQ = 128;       // query rows per tile = UMMA M
constexpr int kTiles = 2;      // query tiles per block: they share every key/value block
constexpr int kBK = 64;        // keys per block
constexpr int kKvStages = 4;     // key/value blocks in flight: later blocks are loaded while block j is in the softmax
constexpr int kTcThreads = 96 + kTiles * 128;
constexpr float kLog2eTc = 1.4426950408889634f;

// sizes for head size D (64 or 128): tiles are halves of 64 columns = 128 bytes, the swizzle's row
template <int D>
struct TcSizes {
    static constexpr int kQBytes = kBQ * D * 2;   // per tile: D / 64 halves of 128 rows x 128 B
    static constexpr int kKBytes = kBK * D * 2;   // D / 64 halves of 64 rows x 128 B
    static constexpr int kSmem = kTiles * kQBytes + kKvStages * 2 * kKBytes + 1024 + 256;
};
constexpr int kTmemColsTc = 512;               // S[tile][buffer] at (tile * 2 + buffer) * 64, O[tile] at 256 + tile * 128

enum TcAttnError { kErrAttnLoader = 11, kErrAttnMma = 12, kErrAttnSoftmax = 13 };

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// instruction descriptors: D fp32, A and B bf16; B K-major (scores) or MN-major (values)
__device__ __forceinline__ constexpr uint32_t idesc_tc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(kBQ >> 4) << 24);
}

template <int kD>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                            int table_stride, const int* __restrict__ positions, const int* __restrict__ qo_indptr,
                            const int* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int o_stride, int nq, int nkv,
                            int page_size, float scale, int* __restrict__ error_flag) {
    ns_pdl_launch_dependents();
    constexpr int kQBytes = TcSizes<kD>::kQBytes, kKBytes = TcSizes<kD>::kKBytes;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t q_smem = base;                                   // [tile]
    const uint32_t kv_smem = q_smem + kTiles * kQBytes;             // [stage][K | V]
    const uint32_t bar0 = kv_smem + kKvStages * 2 * kKBytes;
    // barriers: q_full, kv_full[stage], kv_empty[stage], then per tile s_full[2], s_free[2], p_ready[2], o_done, o_final
    const uint32_t q_full = bar0;
    auto kv_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto kv_empty = [&](int s) { return bar0 + 8u * (1 + kKvStages + s); };
    auto tile_bar = [&](int t, int which) { return bar0 + 8u * (1 + 2 * kKvStages + t * 8 + which); };
    auto s_full = [&](int t, int b) { return tile_bar(t, b); };
    auto s_free = [&](int t, int b) { return tile_bar(t, 2 + b); };
    auto p_ready = [&](int t, int b) { return tile_bar(t, 4 + b); };
    auto o_done = [&](int t) { return tile_bar(t, 6); };
    // Completed once, by the product of the tile's last block.  The output must not be read on o_done's parity: a
    // softmax warp may finish its last block while the product of the block before it is still waiting for the
    // tile's slower warps, and a parity wait two phases ahead of the barrier returns at once.
    auto o_final = [&](int t) { return tile_bar(t, 7); };
    const uint32_t holder = bar0 + 8u * (1 + 2 * kKvStages + kTiles * 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heads vary fastest: the host lists the tiles with the most keys first, and blocks are
    // scheduled in that order, so the long tiles do not end up alone at the tail
    const int req = tiles[2 * blockIdx.y], q_off = tiles[2 * blockIdx.y + 1];
    const int h = blockIdx.x;
    const int hk = h / (nq / nkv);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
        }
        for (int t = 0; t < kTiles; ++t) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(s_full(t, b), 1);
                mbar_init(s_free(t, b), 1);
                mbar_init(p_ready(t, b), 128);
            }
            mbar_init(o_done(t), 1);
            mbar_init(o_final(t), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) tmem_alloc(holder, kTmemColsTc);
    ns_pdl_wait();  // everything below reads what earlier kernels wrote (q, the cache, the step's description)
    const int tok0 = qo_indptr[req] + q_off;
    const int rows_all = min(kTiles * kBQ, qo_indptr[req + 1] - tok0);
    const int pos0 = positions[tok0];
    // per tile: its valid rows and the number of key blocks its last row sees (0 rows: the tile is idle)
    int rows_t[kTiles], nblk_t[kTiles];
    int n_blocks = 0;
#pragma unroll
    for (int t = 0; t < kTiles; ++t) {
        rows_t[t] = max(0, min(kBQ, rows_all - t * kBQ));
        nblk_t[t] = rows_t[t] > 0 ? (pos0 + t * kBQ + rows_t[t] + kBK - 1) / kBK : 0;
        n_blocks = max(n_blocks, nblk_t[t]);
    }
    const int* bt = block_table + (size_t)req * table_stride;
    const int last_blk = (pos0 + rows_all - 1) / page_size;  // the last page that holds one of the keys seen here
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(holder));
    auto tmem_s = [&](int t, int b) { return tmem_base + (uint32_t)((t * 2 + b) * 64); };
    auto tmem_o = [&](int t) { return tmem_base + 256u + (uint32_t)(t * 128); };

    if (warp == 0) {
        // ---------------- loader: the warp runs the loop, one elected lane issues ----------------
        if (elect_one()) {
            mbar_expect_tx(q_full, kTiles * kQBytes);
            for (int t = 0; t < kTiles; ++t) {  // rows past the step's tokens are zero-filled by TMA
#pragma unroll
                for (int hh = 0; hh < kD / 64; ++hh)
                    tma_load_2d(q_smem + t * kQBytes + hh * (kBQ * 128), &map_q, h * kD + hh * 64, tok0 + t * kBQ, q_full);
            }
        }
        const int pages_per_block = kBK / page_size;
        for (int j = 0; j < n_blocks; ++j) {
            const int s = j % kKvStages;
            if (!mbar_wait_warp(kv_empty(s), ((uint32_t)(j / kKvStages) & 1u) ^ 1u)) { if (lane == 0) atomicExch(error_flag, kErrAttnLoader); break; }
            if (elect_one()) mbar_expect_tx(kv_full(s), 2 * kKBytes);
            const uint32_t k_dst = kv_smem + s * 2 * kKBytes, v_dst = k_dst + kKBytes;
            for (int i = 0; i < pages_per_block; ++i) {
                // pages past the last key repeat the last page: finite values that the mask hides
                const int blk = min(j * pages_per_block + i, last_blk);
                const int row = (bt[blk] * nkv + hk) * page_size;
                const uint32_t off = (uint32_t)(i * page_size) * 128u;
                if (elect_one()) {
#pragma unroll
                    for (int hh = 0; hh < kD / 64; ++hh) {
                        tma_load_2d(k_dst + hh * (kBK * 128) + off, &map_k, hh * 64, row, kv_full(s));
                        tma_load_2d(v_dst + hh * (kBK * 128) + off, &map_v, hh * 64, row, kv_full(s));
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- issuer of S = Q K^T: the warp runs the loop, one elected lane issues ----------------
        // tcgen05.mma issue blocks until the tensor core has taken the instruction, so a warp that also
        // waited for the softmax would leave the tensor core idle meanwhile: the two products have a warp each.
        constexpr uint32_t idesc_s = idesc_tc(kBK, false);
        bool ok = mbar_wait_warp(q_full, 0);
        for (int j = 0; ok && j < n_blocks; ++j) {
            const int s = j % kKvStages, b = j & 1;
            // Three things must hold before the scores of block j are issued: its keys have landed, and for each
            // tile S[t][b] is free (it held P of block j-2, and the product that read it is done).  One lane each
            // polls one of the barriers, so the warp pays one wait, not three.
            {
                // the same instructions for the three lanes, with a barrier each
                const int tile = lane == 1 ? 0 : 1;
                const bool frees = lane >= 1 && lane <= kTiles && j >= 2 && j < (tile == 0 ? nblk_t[0] : nblk_t[1]);
                const uint32_t bar = lane == 0 ? kv_full(s) : s_free(tile, b);
                const uint32_t par = lane == 0 ? ((uint32_t)(j / kKvStages) & 1u) : (((uint32_t)(j >> 1) & 1u) ^ 1u);
                bool mine = true;
                if (lane == 0 || frees) mine = mbar_wait(bar, par);
                if (!__all_sync(0xffffffffu, mine)) { ok = false; break; }
            }
            tc_fence_after();
            const uint32_t k_src = kv_smem + s * 2 * kKBytes;
            for (int t = 0; t < kTiles; ++t) {
                if (j >= nblk_t[t]) continue;
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t qa = q_smem + t * kQBytes + (kk >> 2) * (kBQ * 128) + (kk & 3) * 32;
                    const uint32_t kb = k_src + (kk >> 2) * (kBK * 128) + (kk & 3) * 32;
                    if (elect_one()) umma_bf16(tmem_s(t, b), smem_desc(qa), smem_desc(kb), idesc_s, kk > 0 ? 1u : 0u);
                }
                if (elect_one()) umma_commit(s_full(t, b));
            }
        }
        if (!ok && lane == 0) atomicExch(error_flag, kErrAttnMma);
    } else if (warp == 2) {
        // ---------------- issuer of O += P V ----------------
        constexpr uint32_t idesc_o = idesc_tc(kD, true);
        bool ok = true;
        for (int j = 0; ok && j < n_blocks; ++j) {
            const int s = j % kKvStages, b = j & 1;
            const uint32_t v_src = kv_smem + s * 2 * kKBytes + kKBytes;
            for (int t = 0; t < kTiles && ok; ++t) {
                if (j >= nblk_t[t]) continue;
                if (!mbar_wait_warp(p_ready(t, b), (uint32_t)(j >> 1) & 1u)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)  // 16 keys = 8 columns of bf16 pairs
                    if (elect_one())
                        umma_bf16_ts(tmem_o(t), tmem_s(t, b) + kk * 8, smem_desc_mn(v_src + kk * 16 * 128, kBK * 128, 1024),
                                     idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                if (elect_one()) {
                    umma_commit(o_done(t));      // this tile's accumulator holds blocks 0..j
                    umma_commit(s_free(t, b));   // and S[t][b] may take the scores of block j+2
                    if (j == nblk_t[t] - 1) umma_commit(o_final(t));  // the tile's accumulator is complete
                }
            }
            // The stage's values have been read by every tile; its keys were read by the scores of block j,
            // which were complete before the softmax that made P could start.
            if (ok && elect_one()) umma_commit(kv_empty(s));
        }
        if (!ok && lane == 0) atomicExch(error_flag, kErrAttnMma);
    } else if (warp >= 3) {
        // ---------------- softmax and output: one query row per thread, one warpgroup per tile ----------------
        const int t = (warp - 3) >> 2;                             // the tile this warpgroup serves
        const int quarter = warp & 3;                              // the TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;                       // TMEM lane = query row of the tile
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int rows = rows_t[t], my_blocks = nblk_t[t];
        const int tile_pos0 = pos0 + t * kBQ;
        const int pos_row = tile_pos0 + min(row, max(rows, 1) - 1);
        const float sl = scale * kLog2eTc;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < my_blocks; ++j) {
            const int b = j & 1;
            ok = mbar_wait_warp(s_full(t, b), (uint32_t)(j >> 1) & 1u);
            if (!ok) break;
            tc_fence_after();
            uint32_t sv[2][32];
            tmem_ld32(tmem_s(t, b) + lane_addr, sv[0]);
            tmem_ld32(tmem_s(t, b) + lane_addr + 32, sv[1]);
            tmem_ld_wait();
            const int key0 = j * kBK;
            const bool masked = key0 + kBK - 1 > tile_pos0;         // some row of the tile does not see the whole block
            // maximum of the raw scores first (the scale is positive, so it commutes with the maximum),
            // then each weight is one fused multiply-add and one ex2
            if (masked) {
#pragma unroll
                for (int c = 0; c < kBK; ++c)
                    if (key0 + c > pos_row) sv[c >> 5][c & 31] = 0xff800000u;  // -inf
            }
            // eight independent chains: one chain of 64 dependent maxima costs 64 instruction latencies
            float mx8[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) mx8[c] = __uint_as_float(sv[0][c]);
#pragma unroll
            for (int c = 8; c < kBK; ++c) mx8[c & 7] = fmaxf(mx8[c & 7], __uint_as_float(sv[c >> 5][c & 31]));
            const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            // The reference point m of the exponents follows the running maximum lazily: it moves only
            // when the maximum has grown by more than 8 (a factor 256), so the accumulator is rarely
            // rescaled; weights up to 256 are exact enough in bf16 and the sums are fp32.  Block 0
            // holds key 0, so m is finite from the start.
            const float cand = mx * sl;
            const bool jump = cand > m + 8.f;
            const float m_new = jump ? cand : m;
            const float corr = jump ? ex2(m - m_new) : 1.f;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            // weights as bf16 pairs over the first 32 columns of this row's scores
            uint32_t pk[32];
#pragma unroll
            for (int u = 0; u < kBK / 2; ++u) {
                const int c = 2 * u;
                const float p0 = ex2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), sl, -m_new));
                const float p1 = ex2(fmaf(__uint_as_float(sv[(c + 1) >> 5][(c + 1) & 31]), sl, -m_new));
                sum4[u & 3] += p0 + p1;
                __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                pk[u] = *reinterpret_cast<uint32_t*>(&v);
            }
            tmem_st32(tmem_s(t, b) + lane_addr, pk);
            l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            if (j > 0 && __any_sync(0xffffffffu, jump)) {
                // Some row's reference point moved: this warp's rows of the accumulator are rescaled.  They
                // must hold block j-1 first; block j is not added before this warp has arrived below, so
                // the barrier cannot be a phase further.
                ok = mbar_wait_warp(o_done(t), (uint32_t)(j - 1) & 1u);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < kD; c0 += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem_o(t) + lane_addr + c0, ov);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    tmem_st32(tmem_o(t) + lane_addr + c0, ov);
                }
            }
            m = m_new;
            tmem_st_wait();                                         // P (and a rescaled O) are in TMEM
            tc_fence_before();
            mbar_arrive(p_ready(t, b));
        }
        if (ok && my_blocks > 0) ok = mbar_wait_warp(o_final(t), 0);
        if (!ok) {
            if (lane == 0) atomicExch(error_flag, kErrAttnSoftmax);
        } else if (my_blocks > 0) {
            tc_fence_after();
            const float inv = 1.f / l;
            __nv_bfloat16* orow = out + (size_t)(tok0 + t * kBQ + row) * o_stride + (size_t)h * kD;
#pragma unroll 1
            for (int c0 = 0; c0 < kD; c0 += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem_o(t) + lane_addr + c0, ov);
                tmem_ld_wait();
                if (row < rows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 u;
                        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
                        for (int w = 0; w < 4; ++w)
                            hp[w] = __floats2bfloat162_rn(__uint_as_float(ov[i + 2 * w]) * inv, __uint_as_float(ov[i + 2 * w + 1]) * inv);
                        *reinterpret_cast<uint4*>(orow + c0 + i) = u;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemColsTc);
    }
}

// ---------------------------------------------------------------------------------------------------
// Head size 64, an even number of query heads per kv head: one block = 256 query tokens of TWO query heads
// that share a kv head, i.e. four tiles of 128 rows on one stream of keys and values.  With heads of 64 the
// products of a 64-key block need half the tensor-core time of heads of 128 while the softmax costs the
// same, so the kernel above is bound by the exponentials and by the chain scores -> softmax -> P V of its two
// tiles.  Four tiles put four softmax warps on every sub-partition, which keeps its exponential unit busy
// while other warps wait, load or store; TMEM holds them with one buffer of scores per tile (4 x 64 columns
// of S, with P over their first half, and 4 x 64 of O), so a tile's scores of block j+1 follow its P V of
// block j, and the other three tiles fill the tensor core meanwhile.
// The accumulator is up to date whenever a tile's scores arrive (they were issued after its last P V had
// completed), so a rescale needs no barrier.
constexpr int kTiles4 = 4;
constexpr int kTc4Threads = 96 + kTiles4 * 128;
constexpr int kSmem4 = kTiles4 * kBQ * 64 * 2 + kKvStages * 2 * kBK * 64 * 2 + 1024 + 512;

__global__ void __launch_bounds__(kTc4Threads, 1)
attention_prefill_tc4_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                             int table_stride, const int* __restrict__ positions, const int* __restrict__ qo_indptr,
                             const int* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int o_stride, int nq, int nkv,
                             int page_size, float scale, int* __restrict__ error_flag) {
    ns_pdl_launch_dependents();
    constexpr int kD = 64;
    constexpr int kQBytes = kBQ * kD * 2, kKBytes = kBK * kD * 2;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t q_smem = base;                                   // [tile]
    const uint32_t kv_smem = q_smem + kTiles4 * kQBytes;            // [stage][K | V]
    const uint32_t bar0 = kv_smem + kKvStages * 2 * kKBytes;
    // barriers: q_full, kv_full[stage], kv_empty[stage], then per tile s_full, s_free, p_ready, o_final
    const uint32_t q_full = bar0;
    auto kv_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto kv_empty = [&](int s) { return bar0 + 8u * (1 + kKvStages + s); };
    auto tile_bar = [&](int tt, int which) { return bar0 + 8u * (1 + 2 * kKvStages + tt * 4 + which); };
    auto s_full = [&](int tt) { return tile_bar(tt, 0); };   // the scores of the tile's next block are in TMEM
    auto s_free = [&](int tt) { return tile_bar(tt, 1); };   // the P V that read P (over the scores) has completed
    auto p_ready = [&](int tt) { return tile_bar(tt, 2); };  // the 128 softmax threads have stored P
    auto o_final = [&](int tt) { return tile_bar(tt, 3); };  // the P V of the tile's last block has completed
    const uint32_t holder = bar0 + 8u * (1 + 2 * kKvStages + kTiles4 * 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int req = tiles[2 * blockIdx.y], q_off = tiles[2 * blockIdx.y + 1];
    const int h0 = 2 * blockIdx.x;          // tiles 0, 1: head h0; tiles 2, 3: head h0 + 1 (the same kv head)
    const int hk = h0 / (nq / nkv);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
        }
        for (int tt = 0; tt < kTiles4; ++tt) {
            mbar_init(s_full(tt), 1);
            mbar_init(s_free(tt), 1);
            mbar_init(p_ready(tt), 128);
            mbar_init(o_final(tt), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) tmem_alloc(holder, kTmemColsTc);
    ns_pdl_wait();  // everything below reads what earlier kernels wrote (q, the cache, the step's description)
    const int tok0 = qo_indptr[req] + q_off;
    const int rows_all = min(2 * kBQ, qo_indptr[req + 1] - tok0);
    const int pos0 = positions[tok0];
    // per row tile (tile & 1): its valid rows and the number of key blocks its last row sees (0 rows: idle)
    int rows_t[2], nblk_t[2];
    int n_blocks = 0;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        rows_t[t] = max(0, min(kBQ, rows_all - t * kBQ));
        nblk_t[t] = rows_t[t] > 0 ? (pos0 + t * kBQ + rows_t[t] + kBK - 1) / kBK : 0;
        n_blocks = max(n_blocks, nblk_t[t]);
    }
    const int* bt = block_table + (size_t)req * table_stride;
    const int last_blk = (pos0 + rows_all - 1) / page_size;  // the last page that holds one of the keys seen here
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(holder));
    auto tmem_s = [&](int tt) { return tmem_base + (uint32_t)(tt * 64); };
    auto tmem_o = [&](int tt) { return tmem_base + 256u + (uint32_t)(tt * 64); };

    if (warp == 0) {
        // ---------------- loader ----------------
        if (elect_one()) {
            mbar_expect_tx(q_full, kTiles4 * kQBytes);
            for (int tt = 0; tt < kTiles4; ++tt)  // rows past the step's tokens are zero-filled by TMA
                tma_load_2d(q_smem + tt * kQBytes, &map_q, (h0 + (tt >> 1)) * kD, tok0 + (tt & 1) * kBQ, q_full);
        }
        const int pages_per_block = kBK / page_size;
        for (int j = 0; j < n_blocks; ++j) {
            const int s = j % kKvStages;
            if (!mbar_wait_warp(kv_empty(s), ((uint32_t)(j / kKvStages) & 1u) ^ 1u)) { if (lane == 0) atomicExch(error_flag, kErrAttnLoader); break; }
            if (elect_one()) mbar_expect_tx(kv_full(s), 2 * kKBytes);
            const uint32_t k_dst = kv_smem + s * 2 * kKBytes, v_dst = k_dst + kKBytes;
            for (int i = 0; i < pages_per_block; ++i) {
                // pages past the last key repeat the last page: finite values that the mask hides
                const int blk = min(j * pages_per_block + i, last_blk);
                const int row = (bt[blk] * nkv + hk) * page_size;
                const uint32_t off = (uint32_t)(i * page_size) * 128u;
                if (elect_one()) {
                    tma_load_2d(k_dst + off, &map_k, 0, row, kv_full(s));
                    tma_load_2d(v_dst + off, &map_v, 0, row, kv_full(s));
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- issuer of S = Q K^T ----------------
        constexpr uint32_t idesc_s = idesc_tc(kBK, false);
        bool ok = mbar_wait_warp(q_full, 0);
        for (int j = 0; ok && j < n_blocks; ++j) {
            const int s = j % kKvStages;
            ok = mbar_wait_warp(kv_full(s), (uint32_t)(j / kKvStages) & 1u);
            const uint32_t k_src = kv_smem + s * 2 * kKBytes;
            for (int tt = 0; ok && tt < kTiles4; ++tt) {
                if (j >= nblk_t[tt & 1]) continue;
                // the tile's one buffer holds P of block j-1 until the product that reads it has completed
                if (j > 0) ok = mbar_wait_warp(s_free(tt), (uint32_t)(j - 1) & 1u);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk)
                    if (elect_one())
                        umma_bf16(tmem_s(tt), smem_desc(q_smem + tt * kQBytes + kk * 32), smem_desc(k_src + kk * 32), idesc_s,
                                  kk > 0 ? 1u : 0u);
                if (elect_one()) umma_commit(s_full(tt));
            }
        }
        if (!ok && lane == 0) atomicExch(error_flag, kErrAttnMma);
    } else if (warp == 2) {
        // ---------------- issuer of O += P V ----------------
        constexpr uint32_t idesc_o = idesc_tc(kD, true);
        bool ok = true;
        for (int j = 0; ok && j < n_blocks; ++j) {
            const int s = j % kKvStages;
            const uint32_t v_src = kv_smem + s * 2 * kKBytes + kKBytes;
            for (int tt = 0; ok && tt < kTiles4; ++tt) {
                if (j >= nblk_t[tt & 1]) continue;
                ok = mbar_wait_warp(p_ready(tt), (uint32_t)j & 1u);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)  // 16 keys = 8 columns of bf16 pairs
                    if (elect_one())
                        umma_bf16_ts(tmem_o(tt), tmem_s(tt) + kk * 8, smem_desc_mn(v_src + kk * 16 * 128, kBK * 128, 1024),
                                     idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                if (elect_one()) {
                    umma_commit(s_free(tt));                                    // the buffer may take the scores of block j+1
                    if (j == nblk_t[tt & 1] - 1) umma_commit(o_final(tt));      // the tile's accumulator is complete
                }
            }
            // every tile has read the stage's values; its keys were read by the scores of block j
            if (ok && elect_one()) umma_commit(kv_empty(s));
        }
        if (!ok && lane == 0) atomicExch(error_flag, kErrAttnMma);
    } else {
        // ---------------- softmax and output: one query row per thread, one warpgroup per tile ----------------
        const int tt = (warp - 3) >> 2;                            // the tile this warpgroup serves
        const int t = tt & 1;                                      // its rows: the first or the second 128 of the block
        const int h = h0 + (tt >> 1);
        const int quarter = warp & 3;                              // the TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;                       // TMEM lane = query row of the tile
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int rows = rows_t[t], my_blocks = nblk_t[t];
        const int tile_pos0 = pos0 + t * kBQ;
        const int pos_row = tile_pos0 + min(row, max(rows, 1) - 1);
        const float sl = scale * kLog2eTc;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < my_blocks; ++j) {
            ok = mbar_wait_warp(s_full(tt), (uint32_t)j & 1u);
            if (!ok) break;
            tc_fence_after();
            uint32_t sv[2][32];
            tmem_ld32(tmem_s(tt) + lane_addr, sv[0]);
            tmem_ld32(tmem_s(tt) + lane_addr + 32, sv[1]);
            tmem_ld_wait();
            const int key0 = j * kBK;
            if (key0 + kBK - 1 > tile_pos0) {                       // some row of the tile does not see the whole block
#pragma unroll
                for (int c = 0; c < kBK; ++c)
                    if (key0 + c > pos_row) sv[c >> 5][c & 31] = 0xff800000u;  // -inf
            }
            float mx8[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) mx8[c] = __uint_as_float(sv[0][c]);
#pragma unroll
            for (int c = 8; c < kBK; ++c) mx8[c & 7] = fmaxf(mx8[c & 7], __uint_as_float(sv[c >> 5][c & 31]));
            const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            // the reference point follows the maximum lazily, as in the kernel above
            const float cand = mx * sl;
            const bool jump = cand > m + 8.f;
            const float m_new = jump ? cand : m;
            const float corr = jump ? ex2(m - m_new) : 1.f;
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            // the weights of columns 2u and 2u+1 go, as a bf16 pair, where score u lay: it has been used by then
#pragma unroll
            for (int u = 0; u < kBK / 2; ++u) {
                const int c = 2 * u;
                const float p0 = ex2(fmaf(__uint_as_float(sv[c >> 5][c & 31]), sl, -m_new));
                const float p1 = ex2(fmaf(__uint_as_float(sv[(c + 1) >> 5][(c + 1) & 31]), sl, -m_new));
                sum4[u & 3] += p0 + p1;
                __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                sv[0][u] = *reinterpret_cast<uint32_t*>(&v);
            }
            tmem_st32(tmem_s(tt) + lane_addr, sv[0]);
            l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            if (j > 0 && __any_sync(0xffffffffu, jump)) {
                // the accumulator holds blocks 0..j-1: this block's scores were issued after that product completed
#pragma unroll 1
                for (int c0 = 0; c0 < kD; c0 += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem_o(tt) + lane_addr + c0, ov);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                    tmem_st32(tmem_o(tt) + lane_addr + c0, ov);
                }
            }
            m = m_new;
            tmem_st_wait();                                         // P (and a rescaled O) are in TMEM
            tc_fence_before();
            mbar_arrive(p_ready(tt));
        }
        if (ok && my_blocks > 0) ok = mbar_wait_warp(o_final(tt), 0);
        if (!ok) {
            if (lane == 0) atomicExch(error_flag, kErrAttnSoftmax);
        } else if (my_blocks > 0) {
            tc_fence_after();
            const float inv = 1.f / l;
            __nv_bfloat16* orow = out + (size_t)(tok0 + t * kBQ + row) * o_stride + (size_t)h * kD;
#pragma unroll 1
            for (int c0 = 0; c0 < kD; c0 += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem_o(tt) + lane_addr + c0, ov);
                tmem_ld_wait();
                if (row < rows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 u;
                        __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
                        for (int w = 0; w < 4; ++w)
                            hp[w] = __floats2bfloat162_rn(__uint_as_float(ov[i + 2 * w]) * inv, __uint_as_float(ov[i + 2 * w + 1]) * inv);
                        *reinterpret_cast<uint4*>(orow + c0 + i) = u;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemColsTc);
    }
}

template <int kD>
int launch_prefill_tc(const void* q, int q_stride, int n_tokens, const void* k_cache, const void* v_cache, long long n_pages,
                      const int* block_table, int table_stride, const int* positions, const int* qo_indptr, const int* tiles,
                      int n_tiles, void* out, int o_stride, int nq, int nkv, int page_size, float scale, int heads_per_block,
                      int* error_flag, cudaStream_t stream) {
    CUtensorMap mq, mk, mv;
    int rc = ns_make_map_bf16(&mq, q, (unsigned long long)n_tokens, nq * kD, q_stride, kBQ, "ns_attention_prefill_tc");
    if (rc) return rc;
    const unsigned long long cache_rows = (unsigned long long)n_pages * nkv * page_size;
    rc = ns_make_map_bf16(&mk, k_cache, cache_rows, kD, kD, page_size, "ns_attention_prefill_tc");
    if (rc) return rc;
    rc = ns_make_map_bf16(&mv, v_cache, cache_rows, kD, kD, page_size, "ns_attention_prefill_tc");
    if (rc) return rc;
    if (kD == 64 && heads_per_block == 2) {
        static bool configured4 = false;
        if (!configured4) {
            NS_CUDA(cudaFuncSetAttribute(attention_prefill_tc4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem4));
            configured4 = true;
        }
        NS_LAUNCH(attention_prefill_tc4_kernel, dim3(nq / 2, n_tiles), kTc4Threads, kSmem4, stream, mq, mk, mv, block_table,
                  table_stride, positions, qo_indptr, tiles, (__nv_bfloat16*)out, o_stride, nq, nkv, page_size, scale, error_flag);
        NS_CHECK_LAUNCH("ns_attention_prefill_tc");
        return NS_OK;
    }
    static bool configured = false;
    if (!configured) {
        NS_CUDA(cudaFuncSetAttribute(attention_prefill_tc_kernel<kD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     TcSizes<kD>::kSmem));
        configured = true;
    }
    NS_LAUNCH((attention_prefill_tc_kernel<kD>), dim3(nq, n_tiles), kTcThreads, TcSizes<kD>::kSmem, stream, mq, mk, mv,
              block_table, table_stride, positions, qo_indptr, tiles, (__nv_bfloat16*)out, o_stride, nq, nkv, page_size,
              scale, error_flag);
    NS_CHECK_LAUNCH("ns_attention_prefill_tc");
    return NS_OK;
}

}  // namespace

// q: the step's packed projection (bf16, row stride q_stride elements, n_tokens rows); k_cache, v_cache: one
// lane's pages [n_pages, nkv, page_size, head_dim]; tiles: int32 [n_tiles, 2] = (request, offset among its tokens of
// this step, a multiple of 256).  Head sizes 64 and 128; page sizes 8, 16, 32, 64; out rows 16-byte aligned.
// heads_per_block: 1, or 2 for heads of 64 in groups of an even size (two query heads of a kv head share a block and
// its stream of keys and values: worth it once there are more blocks than SMs).
NS_API int ns_attention_prefill_tc(const void* q, int q_stride, int n_tokens, const void* k_cache, const void* v_cache,
                                   long long n_pages, const int* block_table, int table_stride, const int* positions,
                                   const int* qo_indptr, const int* tiles, int n_tiles, void* out, int o_stride, int nq,
                                   int nkv, int d, int page_size, float scale, int heads_per_block, int* error_flag,
                                   cudaStream_t stream) {
    if (n_tiles <= 0) return NS_OK;
    if (d != 64 && d != 128) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill_tc: head_dim=%d (64 or 128)", d);
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill_tc: page_size=%d (8, 16, 32 or 64)", page_size);
    if (nkv < 1 || nq % nkv || n_tiles > 65535)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill_tc: %d heads over %d kv heads, %d tiles", nq, nkv, n_tiles);
    if (q_stride % 8 || o_stride % 8 || ((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill_tc: rows must be 16-byte aligned");
    if (heads_per_block != 1 && !(heads_per_block == 2 && d == 64 && (nq / nkv) % 2 == 0))
        NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_prefill_tc: heads_per_block=%d (1, or 2 with heads of 64 in groups of an even size)", heads_per_block);
    if (!error_flag) NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_prefill_tc: no error flag");
    if (d == 64)
        return launch_prefill_tc<64>(q, q_stride, n_tokens, k_cache, v_cache, n_pages, block_table, table_stride, positions,
                                     qo_indptr, tiles, n_tiles, out, o_stride, nq, nkv, page_size, scale, heads_per_block, error_flag, stream);
    return launch_prefill_tc<128>(q, q_stride, n_tokens, k_cache, v_cache, n_pages, block_table, table_stride, positions,
                                  qo_indptr, tiles, n_tiles, out, o_stride, nq, nkv, page_size, scale, heads_per_block, error_flag,
                                  stream);
}
