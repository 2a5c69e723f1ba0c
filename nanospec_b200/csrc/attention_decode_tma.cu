// Decode attention over the paged cache for head sizes 64 and 128 (bfloat16), built for a short
// chain of dependent steps: one query token per request, its keys split over the blocks of a
// thread-block cluster.
//
// Grid (split, kv head x head tile, token), cluster (splits, 1, 1).  In a block, one warp brings
// 64 keys and values at a time from the cache pages into 128-byte-swizzled shared memory with TMA
// (one box of page_size x 64 elements per page and half of the head; an mbarrier per stage counts
// the bytes), and four warps consume them: each takes 16 keys of every tile, computes scores and the
// weighted sum on the tensor cores (m16n8k16, the group's query heads padded to 16 rows, the query
// fragments read straight from global memory), and keeps the softmax in fp32 (online, base 2).
// The loads of all keys but the token's own are issued before the kernel waits for its predecessor in
// the stream (programmatic dependent launch), so the cache streams in while the query is still
// being rotated.  No block-wide barrier inside the loop: a warp waits for the tile's mbarrier and gives the stage
// back through another.  At the end the four warps' partial results are combined in shared memory,
// and the blocks of the cluster combine theirs through distributed shared memory: every block owns
// one slice of the output, the others store their share of it into its shared memory, and after one
// cluster barrier it adds them in split order - no scratch in global memory, no atomics, and a
// result that does not depend on timing.  Launch dimensions do not depend on sequence lengths.
//
// A batch whose contexts differ much in length would leave the blocks of the longest request streaming alone long
// after the others are done.  The host therefore may hand the kernel a work list instead of rows: items (token row,
// request, keys the request sees, group) in which a long request appears several times, each time for a part of its
// keys.  A cluster then stores its result unnormalised (with the maxima and sums) in global memory, counts itself
// in, and the block that finds the request's other parts complete adds them up in the order of the parts.  An item
// holds all that the kernel otherwise reads from the step's description, one load instead of a chain of three.
//
// Tokens whose request brings more than one token are left to the prefill kernel; padding rows
// (request index < 0) are skipped.  Page sizes 8, 16, 32, 64.  Every mbarrier wait is bounded; a
// wait that runs out sets *error_flag and the block winds down through the same barriers.
#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"

namespace {

constexpr int kKeys = 64;            // keys per tile
constexpr int kComputeWarps = 4;
constexpr int kDtThreads = (kComputeWarps + 1) * 32;
// tiles of 64 keys in flight per block: 96 KB of keys and values for either head size, two blocks per SM
template <int D>
constexpr int dt_stages() { return D == 64 ? 6 : 3; }
constexpr int kMaxClusterSplits = 16;
constexpr float kLog2eDt = 1.4426950408889634f;

enum DecodeTmaError { kErrDecodeLoader = 21, kErrDecodeCompute = 22 };

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// 16 bytes at (row, col) of a tile stored as halves of 64 rows x 128 bytes with the 128-byte swizzle;
// col is a multiple of 8 elements
__device__ __forceinline__ uint32_t swizzled(uint32_t tile, int row, int col) {
    return tile + (uint32_t)(col >> 6) * (kKeys * 128) + (uint32_t)row * 128u +
           (uint32_t)((((col & 63) >> 3) ^ (row & 7)) << 4);
}

// one part of a request that the work list has cut up, per (kv head, head tile): [16 rows][D] sums, then [16][maximum, sum]
template <int D>
constexpr int kPartFloats = 16 * D + 32;

// Every block that has stored its share of a part counts itself in; the one that completes the count (parts x splits
// blocks) finds all the parts in global memory and adds them up in the order of the parts.  The counter goes back to
// zero for the next launch.
template <int D>
__device__ __forceinline__ void merge_parts(const float* part, int* counters, int meta, int n_splits, __nv_bfloat16* out_row,
                                            int total) {
    __shared__ int last;
    const int first = meta >> 8, parts = meta & 15;
    __threadfence();       // this thread's stores are visible before the count below
    __syncthreads();
    int* counter = counters + (size_t)first * gridDim.y + blockIdx.y;
    if (threadIdx.x == 0) last = atomicAdd(counter, 1) == parts * n_splits - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();       // the other blocks' stores, counted before this block's, are visible to the loads below
    const float* p0 = part + ((size_t)first * gridDim.y + blockIdx.y) * kPartFloats<D>;
    const size_t stride = (size_t)gridDim.y * kPartFloats<D>;
    for (int e = threadIdx.x; e < total; e += kDtThreads) {
        const int row = e / D;
        float mt = -INFINITY;
        for (int c = 0; c < parts; ++c) mt = fmaxf(mt, __ldcg(p0 + c * stride + 16 * D + 2 * row));
        float acc = 0.f, lt = 0.f;
        for (int c = 0; c < parts; ++c) {
            const float ms = __ldcg(p0 + c * stride + 16 * D + 2 * row);
            const float f = ms == -INFINITY ? 0.f : ns_exp2(ms - mt);
            acc += __ldcg(p0 + c * stride + e) * f;
            lt += __ldcg(p0 + c * stride + 16 * D + 2 * row + 1) * f;
        }
        out_row[e] = __float2bfloat16_rn(acc / lt);
    }
    if (threadIdx.x == 0) *counter = 0;
}

template <int D>
__global__ void __launch_bounds__(kDtThreads, 2)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __nv_bfloat16* __restrict__ q, int q_stride, const int* __restrict__ block_table,
                            int table_stride, const int* __restrict__ token_req, const int* __restrict__ positions,
                            const int* __restrict__ qo_indptr, __nv_bfloat16* __restrict__ out, int o_stride,
                            const int* __restrict__ rows, int nq, int nkv, int page_size, float scale, int window,
                            int head_tiles, int* __restrict__ error_flag, const int4* __restrict__ work,
                            float* __restrict__ part, int* __restrict__ counters) {
    ns_pdl_launch_dependents();
    constexpr int kDtStages = dt_stages<D>();
    constexpr int kTileBytes = kKeys * D * 2;      // the keys or the values of one tile
    constexpr int kStageBytes = 2 * kTileBytes;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_dyn + (base - smem_u32(smem_dyn));
    // what the other blocks of the cluster send here: [split][elements of this block's slice], then
    // [split][16 rows][maximum, sum]
    float* recv_o = reinterpret_cast<float*>(base_ptr + kDtStages * kStageBytes);
    float* recv_ml = recv_o + 16 * D + kMaxClusterSplits;
    const uint32_t recv_o_addr = base + kDtStages * kStageBytes;
    const uint32_t recv_ml_addr = recv_o_addr + (16 * D + kMaxClusterSplits) * 4;
    const uint32_t bar0 = recv_ml_addr + kMaxClusterSplits * 32 * 4;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kDtStages + s); };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kDtStages; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), kComputeWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    __syncthreads();
    // The step's description and every key but the newest were written before this step's kernels
    // started: by the copy that opens every step (a stream operation, which programmatic launches never
    // overlap - so all of the previous step is complete and visible when any kernel of this step runs), or
    // by earlier steps.  They are read before this kernel waits for its predecessor.  Only the query and
    // the tile that holds the token's own key (written earlier in this step) come after the wait.

    const int n_splits = gridDim.x, split = blockIdx.x, z = blockIdx.z;
    // the token this cluster works for; with a work list also its request, the keys it sees and the part of them that
    // this item takes: meta = first slot << 8 | part << 4 | parts, or -1 for a whole request
    int n, req, pos, meta = -1;
    if (work) {
        const int4 item = work[z];
        n = item.x, req = item.y, pos = item.z - 1, meta = item.w;  // an unused item has request -1
    } else {
        n = rows ? rows[z] : z;
        req = token_req[n];
        if (req >= 0 && qo_indptr[req + 1] - qo_indptr[req] != 1) req = -1;  // not a decode row: the prefill kernel's
        pos = req >= 0 ? positions[n] : 0;
    }
    const int hk = blockIdx.y / head_tiles, ht = blockIdx.y - hk * head_tiles;
    // (the same for every block of the cluster; a block with nothing to do still waits for the predecessor, so that
    // a grid of nothing but such blocks cannot complete before it and let its own successor start too early)
    if (req < 0) { ns_pdl_wait(); return; }
    // a block's shared memory may be written by the others only once it runs: every block says so here
    // and checks the others before its first store into them
    if (n_splits > 1) cluster_arrive();
    const int G = nq / nkv;
    const int h0 = hk * G + ht * 16;
    const int gcount = min(16, G - ht * 16);
    int kend = pos + 1;
    int kstart = (window > 0 && kend - window > 0) ? kend - window : 0;
    if (meta >= 0) {
        // part c of `parts`: whole tiles of 64 keys, as the packer counted them
        const int parts = meta & 15, c = (meta >> 4) & 15;
        const int each = (((kend + parts - 1) / parts + kKeys - 1) / kKeys) * kKeys;
        kstart = c * each;
        kend = min(kend, kstart + each);
    }
    const int origin = kstart & ~(kKeys - 1);                  // tiles start on a page edge
    const int chunk = (((kend - origin + n_splits - 1) / n_splits + kKeys - 1) / kKeys) * kKeys;
    const int k0 = origin + split * chunk;
    const int k1 = min(k0 + chunk, kend);
    const int n_tiles = k0 < k1 ? (k1 - k0 + kKeys - 1) / kKeys : 0;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

    if (warp == kComputeWarps) {
        // ---------------- loader: the warp runs the loop, one elected lane issues ----------------
        const int* bt = block_table + (size_t)req * table_stride;
        const int page_shift = 31 - __clz(page_size);
        const int pages_per_tile = kKeys >> page_shift;
        const int first_page = kstart >> page_shift;          // pages before it may have been given back
        const int last_page = (kend - 1) >> page_shift;       // pages past it repeat it: finite values that the mask hides
        bool waited = false;
        for (int t = 0; t < n_tiles; ++t) {
            const int s = t % kDtStages;
            // the tile with the token's own key, and whatever needs a stage back from the other warps (they
            // wait for the query first), come after the wait for the previous kernel
            if (!waited && (t >= kDtStages || k0 + (t + 1) * kKeys > pos)) {
                ns_pdl_wait();
                waited = true;
            }
            if (t >= kDtStages && !mbar_wait_warp(empty(s), (uint32_t)(t / kDtStages - 1) & 1u)) {
                if (lane == 0) atomicExch(error_flag, kErrDecodeLoader);
                break;
            }
            int page = 0;
            if (lane < pages_per_tile) {
                const int p = ((k0 + t * kKeys) >> page_shift) + lane;
                page = bt[min(max(p, first_page), last_page)];
            }
            if (elect_one()) mbar_expect_tx(full(s), kStageBytes);
            const uint32_t k_dst = base + s * kStageBytes, v_dst = k_dst + kTileBytes;
            for (int i = 0; i < pages_per_tile; ++i) {
                const int row = (__shfl_sync(0xffffffffu, page, i) * nkv + hk) * page_size;
                const uint32_t off = (uint32_t)(i * page_size) * 128u;
                if (elect_one()) {
#pragma unroll
                    for (int hh = 0; hh < D / 64; ++hh) {
                        tma_load_2d(k_dst + hh * (kKeys * 128) + off, &map_k, hh * 64, row, full(s));
                        tma_load_2d(v_dst + hh * (kKeys * 128) + off, &map_v, hh * 64, row, full(s));
                    }
                }
            }
        }
    } else {
        // ---------------- four warps: 16 keys of every tile each ----------------
        ns_pdl_wait();  // the query comes from the previous kernel, and nothing is written before it is done
        uint32_t qf[D / 16][4];
        {
            const int g = lane >> 2, c2 = 2 * (lane & 3);
            const __nv_bfloat16* qrow = q + (size_t)n * q_stride + (size_t)h0 * D;
            const bool lo = g < gcount, hi = g + 8 < gcount;  // rows beyond the group are zero
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const __nv_bfloat16* a = qrow + (size_t)g * D + kk * 16 + c2;
                const __nv_bfloat16* b = a + 8 * D;
                qf[kk][0] = lo ? *reinterpret_cast<const uint32_t*>(a) : 0u;
                qf[kk][1] = hi ? *reinterpret_cast<const uint32_t*>(b) : 0u;
                qf[kk][2] = lo ? *reinterpret_cast<const uint32_t*>(a + 8) : 0u;
                qf[kk][3] = hi ? *reinterpret_cast<const uint32_t*>(b + 8) : 0u;
            }
        }
        const float sl = scale * kLog2eDt;
        const int mat = lane >> 3, r8 = lane & 7;
        bool ok = true;
        for (int t = 0; t < n_tiles; ++t) {
            const int s = t % kDtStages;
            if (!mbar_wait_warp(full(s), (uint32_t)(t / kDtStages) & 1u)) { ok = false; break; }
            const uint32_t ks = base + s * kStageBytes, vs = ks + kTileBytes;
            const int kb = k0 + t * kKeys + warp * 16;
            if (kb < k1 && kb + 16 > kstart) {  // some key of the 16 is seen
                float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, swizzled(ks, warp * 16 + (mat >> 1) * 8 + r8, kk * 16 + (mat & 1) * 8));
                    ns_mma_bf16(sc[0], qf[kk], kf[0], kf[1]);
                    ns_mma_bf16(sc[1], qf[kk], kf[2], kf[3]);
                }
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int key = kb + nb * 8 + 2 * (lane & 3) + (j & 1);
                        const float v = (key < k1 && key >= kstart) ? sc[nb][j] * sl : -INFINITY;
                        sc[nb][j] = v;
                        mx[j >> 1] = fmaxf(mx[j >> 1], v);
                    }
                float corr[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                    const float m_new = fmaxf(m[i], mx[i]);  // finite: every row sees the same keys, one of them here
                    corr[i] = ns_exp2(m[i] - m_new);
                    m[i] = m_new;
                    l[i] *= corr[i];
                }
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float p = ns_exp2(sc[nb][j] - m[j >> 1]);
                        sc[nb][j] = p;
                        l[j >> 1] += p;
                    }
                uint32_t pa[4] = {ns_pack_bf16(sc[0][0], sc[0][1]), ns_pack_bf16(sc[0][2], sc[0][3]),
                                  ns_pack_bf16(sc[1][0], sc[1][1]), ns_pack_bf16(sc[1][2], sc[1][3])};
                if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {  // some row's maximum moved
#pragma unroll
                    for (int nb = 0; nb < D / 8; ++nb) {
                        o[nb][0] *= corr[0]; o[nb][1] *= corr[0];
                        o[nb][2] *= corr[1]; o[nb][3] *= corr[1];
                    }
                }
#pragma unroll
                for (int nb2 = 0; nb2 < D / 16; ++nb2) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, swizzled(vs, warp * 16 + (mat & 1) * 8 + r8, nb2 * 16 + (mat >> 1) * 8));
                    ns_mma_bf16(o[2 * nb2], pa, vf[0], vf[1]);
                    ns_mma_bf16(o[2 * nb2 + 1], pa, vf[2], vf[3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty(s));  // this warp is done with the stage
        }
        if (!ok && lane == 0) atomicExch(error_flag, kErrDecodeCompute);
    }

    // ---- combine the four warps (each saw a quarter of every tile): the stages are free now -------
    __syncthreads();
    constexpr int SO = D + 8;                         // padded rows: the warps' stores do not collide
    float* so = reinterpret_cast<float*>(base_ptr);  // [warp][16][SO]
    float* sm = so + kComputeWarps * 16 * SO;         // [warp][16] maximum, then [warp][16] sum
    if (warp < kComputeWarps) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
            l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
        }
        const int r0 = lane >> 2;
        float* mine = so + (size_t)warp * 16 * SO;
        if (r0 < gcount) {                            // rows beyond the group hold nothing
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb)
                *reinterpret_cast<float2*>(mine + (size_t)r0 * SO + nb * 8 + 2 * (lane & 3)) = make_float2(o[nb][0], o[nb][1]);
        }
        if (r0 + 8 < gcount) {
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb)
                *reinterpret_cast<float2*>(mine + (size_t)(r0 + 8) * SO + nb * 8 + 2 * (lane & 3)) = make_float2(o[nb][2], o[nb][3]);
        }
        if ((lane & 3) == 0) {
            sm[warp * 16 + r0] = m[0];
            sm[warp * 16 + r0 + 8] = m[1];
            sm[64 + warp * 16 + r0] = l[0];
            sm[64 + warp * 16 + r0 + 8] = l[1];
        }
    }
    __syncthreads();
    // With several splits every block owns one slice of the output: a block sends each element of its
    // result to the element's owner (a store into the owner's shared memory), its maxima and sums to all.
    const int total = gcount * D;
    const int per = (total + n_splits - 1) / n_splits;  // elements per owner
    if (n_splits > 1) cluster_wait();                    // every block of the cluster has started
    for (int e = tid; e < total; e += kDtThreads) {
        const int row = e / D, col = e - row * D;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < kComputeWarps; ++w) mt = fmaxf(mt, sm[w * 16 + row]);
        float acc = 0.f, lt = 0.f;
        if (mt > -INFINITY) {
#pragma unroll
            for (int w = 0; w < kComputeWarps; ++w) {
                const float f = ns_exp2(sm[w * 16 + row] - mt);
                acc += so[((size_t)w * 16 + row) * SO + col] * f;
                lt += sm[64 + w * 16 + row] * f;
            }
        }
        if (n_splits == 1) {
            if (meta < 0) {
                out[(size_t)n * o_stride + (size_t)(h0 + row) * D + col] = __float2bfloat16_rn(acc / lt);
            } else {
                float* slot = part + ((size_t)((meta >> 8) + ((meta >> 4) & 15)) * gridDim.y + blockIdx.y) * kPartFloats<D>;
                slot[e] = acc;
                if (col == 0) { slot[16 * D + 2 * row] = mt; slot[16 * D + 2 * row + 1] = lt; }
            }
        } else {
            const int owner = e / per;
            st_cluster_f32(recv_o_addr + 4u * (uint32_t)(split * per + (e - owner * per)), (uint32_t)owner, acc);
            if (col == 0) {
                for (int r = 0; r < n_splits; ++r) {
                    st_cluster_f32(recv_ml_addr + 4u * (uint32_t)((split * 16 + row) * 2), (uint32_t)r, mt);
                    st_cluster_f32(recv_ml_addr + 4u * (uint32_t)((split * 16 + row) * 2 + 1), (uint32_t)r, lt);
                }
            }
        }
    }
    if (n_splits == 1) {
        if (meta >= 0) merge_parts<D>(part, counters, meta, n_splits, out + (size_t)n * o_stride + (size_t)h0 * D, total);
        return;
    }

    // ---- one cluster barrier, then every block merges its slice from its own shared memory, in split order ----
    cluster_sync();
    for (int i = tid; i < per && split * per + i < total; i += kDtThreads) {
        const int e = split * per + i;
        const int row = e / D;
        float mt = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < kMaxClusterSplits; ++s2)
            if (s2 < n_splits) mt = fmaxf(mt, recv_ml[(s2 * 16 + row) * 2]);
        float acc = 0.f, lt = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < kMaxClusterSplits; ++s2) {
            if (s2 < n_splits) {
                const float ms = recv_ml[(s2 * 16 + row) * 2];
                const float f = ms == -INFINITY ? 0.f : ns_exp2(ms - mt);  // an empty split adds nothing
                acc += recv_o[s2 * per + i] * f;
                lt += recv_ml[(s2 * 16 + row) * 2 + 1] * f;
            }
        }
        if (meta < 0) {
            out[(size_t)n * o_stride + (size_t)h0 * D + e] = __float2bfloat16_rn(acc / lt);
        } else {
            float* slot = part + ((size_t)((meta >> 8) + ((meta >> 4) & 15)) * gridDim.y + blockIdx.y) * kPartFloats<D>;
            slot[e] = acc;
            if (e - row * D == 0) { slot[16 * D + 2 * row] = mt; slot[16 * D + 2 * row + 1] = lt; }
        }
    }
    // nothing reads another block's shared memory after the barrier: a block may exit when it is done
    if (meta >= 0) merge_parts<D>(part, counters, meta, n_splits, out + (size_t)n * o_stride + (size_t)h0 * D, total);
}

template <int D>
int launch_decode_tma(const CUtensorMap& mk, const CUtensorMap& mv, const void* q, int q_stride, const int* block_table,
                      int table_stride, const int* token_req, const int* positions, const int* qo_indptr, void* out,
                      int o_stride, const int* rows, int n_tokens, int nq, int nkv, int page_size, float scale, int window,
                      int n_splits, int* error_flag, const int* work, float* part, int* counters, cudaStream_t stream) {
    constexpr int kDtStages = dt_stages<D>();
    constexpr int kSmem = kDtStages * 2 * kKeys * D * 2 + (16 * D + kMaxClusterSplits + kMaxClusterSplits * 32) * 4 + 2 * kDtStages * 8 + 1024;
    static_assert(kDtStages * 2 * kKeys * D * 2 >= (kComputeWarps * 16 * (D + 8) + 128) * 4, "the warps' partial results reuse the stages");
    static bool configured = false;
    if (!configured) {
        NS_CUDA(cudaFuncSetAttribute(attention_decode_tma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
        NS_CUDA(cudaFuncSetAttribute(attention_decode_tma_kernel<D>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        configured = true;
    }
    const int head_tiles = (nq / nkv + 15) / 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_splits, nkv * head_tiles, n_tokens);
    cfg.blockDim = dim3(kDtThreads);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (ns_pdl_enabled) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (n_splits > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = n_splits;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    (void)cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel<D>, mk, mv, (const __nv_bfloat16*)q, q_stride, block_table,
                             table_stride, token_req, positions, qo_indptr, (__nv_bfloat16*)out, o_stride, rows, nq, nkv,
                             page_size, scale, window, head_tiles, error_flag, (const int4*)work, part, counters);
    NS_CHECK_LAUNCH("ns_attention_decode_tma");
    return NS_OK;
}

}  // namespace

// bfloat16, head_dim 64 or 128, page sizes 8 to 64; k_cache, v_cache: one lane's pages
// [n_pages, nkv, page_size, head_dim]; n_splits 1, 2, 4, 8 or 16 (the blocks of one cluster).
// `rows` (optional) lists the token rows to work on (n_tokens of them).
// `work` (optional, instead of rows; not with a window): n_tokens items of four ints (token row or -1 for an unused
// item, first key, end key, meta) as the cache manager's packer writes them: a request whose context is much longer
// than the others' appears once per part of its keys, meta = first slot << 8 | part << 4 | parts (at most 15 parts),
// and -1 for a whole request.  `part` then holds (slots) x (kv heads x head tiles) x (16 x head_dim + 32) floats and
// `counters` (slots) x (kv heads x head tiles) ints that are zero before the first launch (the kernel leaves them zero).
NS_API int ns_attention_decode_tma(const void* q, int q_stride, const void* k_cache, const void* v_cache, long long n_pages,
                                   const int* block_table, int table_stride, const int* token_req, const int* positions,
                                   const int* qo_indptr, void* out, int o_stride, const int* rows, int n_tokens, int nq,
                                   int nkv, int d, int page_size, float scale, int window, int n_splits, int* error_flag,
                                   const int* work, float* part, int* counters, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (work && (window > 0 || rows || !part || !counters || (uintptr_t)work % 16))
        NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_decode_tma: a work list goes without rows and without a window, with its scratch, 16-byte aligned");
    if (d != 64 && d != 128) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_tma: head_dim=%d (64 or 128)", d);
    if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_tma: page_size=%d (8, 16, 32 or 64)", page_size);
    if (nkv < 1 || nq % nkv) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_tma: %d query heads over %d kv heads", nq, nkv);
    if (n_splits < 1 || n_splits > kMaxClusterSplits || (n_splits & (n_splits - 1)))
        NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_decode_tma: n_splits=%d (1, 2, 4, 8 or 16)", n_splits);
    if (n_tokens > 65535) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_tma: %d tokens exceed the grid", n_tokens);
    if (q_stride % 2 || ((uintptr_t)q % 4) || ((uintptr_t)k_cache | (uintptr_t)v_cache) % 16)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_tma: q rows must be 4-byte and the cache 16-byte aligned");
    if (!error_flag) NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_decode_tma: no error flag");
    CUtensorMap mk, mv;
    const unsigned long long cache_rows = (unsigned long long)n_pages * nkv * page_size;
    int rc = ns_make_map_bf16(&mk, k_cache, cache_rows, d, d, page_size, "ns_attention_decode_tma");
    if (rc) return rc;
    rc = ns_make_map_bf16(&mv, v_cache, cache_rows, d, d, page_size, "ns_attention_decode_tma");
    if (rc) return rc;
    if (d == 64)
        return launch_decode_tma<64>(mk, mv, q, q_stride, block_table, table_stride, token_req, positions, qo_indptr, out,
                                     o_stride, rows, n_tokens, nq, nkv, page_size, scale, window, n_splits, error_flag, work, part,
                                     counters, stream);
    return launch_decode_tma<128>(mk, mv, q, q_stride, block_table, table_stride, token_req, positions, qo_indptr, out,
                                  o_stride, rows, n_tokens, nq, nkv, page_size, scale, window, n_splits, error_flag, work, part,
                                  counters, stream);
}
