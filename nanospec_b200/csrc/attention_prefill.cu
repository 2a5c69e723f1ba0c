// Prefill attention over the paged cache in bfloat16: portions of prompts (more than one query
// token per request), causal and aligned to absolute positions, so a portion that continues a
// request attends to everything the request has in the cache plus its own earlier tokens.
//
// Grid (query tile, query head).  A query tile is 128 consecutive tokens of one request, given
// by the host as (request, offset into the request's tokens of this step); each of the 8 warps
// owns 16 query rows.  Keys and values of the head's kv head stream through shared memory with
// cp.async in tiles of 64 (two stages); scores and the weighted sum run on the tensor cores
// (m16n8k16), the softmax is online in fp32 (base 2).  A query at position p sees keys
// max(0, p - window + 1) .. p (window 0: all of 0 .. p).
//
// Requests that bring exactly one token are left to the decode kernel; the host lists no tile
// for them.
#include "attention_common.cuh"

namespace {

constexpr int kTileQ = 128;        // query rows per block: 8 warps of 16 rows
constexpr int kPrefillThreads = 256;

template <int D>
__global__ void __launch_bounds__(kPrefillThreads)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                         int table_stride, const int* __restrict__ positions, const int* __restrict__ qo_indptr,
                         const int* __restrict__ tiles, __nv_bfloat16* __restrict__ out, int o_stride, int nq, int nkv,
                         int page_size, float scale, int window) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    using Tile = NsTile<D>;
    constexpr int S = Tile::kStride;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [64][S]
    __nv_bfloat16* kv = qs + kTileQ * S;                              // [stage][k|v][64][S]

    const int req = tiles[2 * blockIdx.x], q_off = tiles[2 * blockIdx.x + 1];
    const int h = blockIdx.y;
    const int hk = h / (nq / nkv);
    const int tok0 = qo_indptr[req] + q_off;
    const int rows = min(kTileQ, qo_indptr[req + 1] - tok0);  // valid query rows of this tile
    const int pos0 = positions[tok0];                         // positions of a request's tokens are consecutive
    const int pos_last = pos0 + rows - 1;
    const int kend = pos_last + 1;
    const int kfirst = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
    const int k_begin = (kfirst / kTileKeys) * kTileKeys;
    const int n_tiles = (kend - k_begin + kTileKeys - 1) / kTileKeys;
    const int* bt = block_table + (size_t)req * table_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

    {
        constexpr int kChunks = D / 8;
        const __nv_bfloat16* qbase = q + (size_t)tok0 * q_stride + (size_t)h * D;
        for (int c = tid; c < kTileQ * kChunks; c += kPrefillThreads) {
            const int row = c / kChunks, ch = c - row * kChunks;
            const bool valid = row < rows;
            ns_cp_async16(Tile::at(qs, row, ch * 8), qbase + (valid ? (size_t)row * q_stride + ch * 8 : 0), valid);
        }
    }
    load_kv_tile<D, kPrefillThreads>(kv, kv + kTileKeys * S, k_cache, v_cache, bt, k_begin, kfirst, kend, hk, nkv, page_size, page_shift);
    ns_cp_async_commit();

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    uint32_t qf[D / 16][4];
    const float sl = scale * kLog2e;
    const int mat = lane >> 3, r8 = lane & 7;
    // this thread's two query rows and their positions (rows past the end repeat the last one)
    int prow[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) prow[i] = pos0 + min(warp * 16 + (lane >> 2) + 8 * i, rows - 1);
    const int warp_pos_max = pos0 + min(warp * 16 + 15, rows - 1);
    const bool warp_active = warp * 16 < rows;

    for (int t = 0; t < n_tiles; ++t) {
        __nv_bfloat16* ks = kv + (size_t)(t & 1) * 2 * kTileKeys * S;
        __nv_bfloat16* vs = ks + kTileKeys * S;
        if (t + 1 < n_tiles) {
            __nv_bfloat16* kn = kv + (size_t)((t + 1) & 1) * 2 * kTileKeys * S;
            load_kv_tile<D, kPrefillThreads>(kn, kn + kTileKeys * S, k_cache, v_cache, bt, k_begin + (t + 1) * kTileKeys, kfirst, kend, hk,
                            nkv, page_size, page_shift);
        }
        ns_cp_async_commit();
        ns_cp_async_wait<1>();
        __syncthreads();
        if (t == 0) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                ns_ldmatrix_x4(qf[kk], Tile::at(qs, warp * 16 + (mat & 1) * 8 + r8, kk * 16 + (mat >> 1) * 8));
        }
        const int kb = k_begin + t * kTileKeys;
        if (warp_active && kb <= warp_pos_max) {  // some key of the tile is visible to some row of the warp
            float s[8][4];
#pragma unroll
            for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[nb][j] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
                for (int nb2 = 0; nb2 < 4; ++nb2) {
                    uint32_t kf[4];
                    ns_ldmatrix_x4(kf, Tile::at(ks, nb2 * 16 + (mat >> 1) * 8 + r8, kk * 16 + (mat & 1) * 8));
                    ns_mma_bf16(s[2 * nb2], qf[kk], kf[0], kf[1]);
                    ns_mma_bf16(s[2 * nb2 + 1], qf[kk], kf[2], kf[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
            // tiles that lie wholly inside every row's visible range need no mask
            const int warp_pos_min = pos0 + min(warp * 16, rows - 1);
            const bool full = kb + kTileKeys - 1 <= warp_pos_min && (window <= 0 || kb > warp_pos_max - window);
            if (full) {
#pragma unroll
                for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float v = s[nb][j] * sl;
                        s[nb][j] = v;
                        mx[j >> 1] = fmaxf(mx[j >> 1], v);
                    }
            } else {
#pragma unroll
                for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int key = kb + nb * 8 + 2 * (lane & 3) + (j & 1);
                        const int p = prow[j >> 1];
                        const bool seen = key <= p && (window <= 0 || key > p - window);
                        const float v = seen ? s[nb][j] * sl : -INFINITY;
                        s[nb][j] = v;
                        mx[j >> 1] = fmaxf(mx[j >> 1], v);
                    }
            }
            float corr[2], m_use[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m[i], mx[i]);
                m_use[i] = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet
                corr[i] = ns_exp2(m[i] - m_use[i]);
                m[i] = m_new;
                l[i] *= corr[i];
            }
#pragma unroll
            for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p = ns_exp2(s[nb][j] - m_use[j >> 1]);
                    s[nb][j] = p;
                    l[j >> 1] += p;
                }
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {  // some row's maximum moved
#pragma unroll
                for (int nb = 0; nb < D / 8; ++nb) {
                    o[nb][0] *= corr[0]; o[nb][1] *= corr[0];
                    o[nb][2] *= corr[1]; o[nb][3] *= corr[1];
                }
            }
#pragma unroll
            for (int kb16 = 0; kb16 < 4; ++kb16) {
                uint32_t pa[4] = {ns_pack_bf16(s[2 * kb16][0], s[2 * kb16][1]), ns_pack_bf16(s[2 * kb16][2], s[2 * kb16][3]),
                                  ns_pack_bf16(s[2 * kb16 + 1][0], s[2 * kb16 + 1][1]),
                                  ns_pack_bf16(s[2 * kb16 + 1][2], s[2 * kb16 + 1][3])};
#pragma unroll
                for (int nb2 = 0; nb2 < D / 16; ++nb2) {
                    uint32_t vf[4];
                    ns_ldmatrix_x4_trans(vf, Tile::at(vs, kb16 * 16 + (mat & 1) * 8 + r8, nb2 * 16 + (mat >> 1) * 8));
                    ns_mma_bf16(o[2 * nb2], pa, vf[0], vf[1]);
                    ns_mma_bf16(o[2 * nb2 + 1], pa, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();
    }
    ns_cp_async_wait<0>();

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = warp * 16 + (lane >> 2) + 8 * i;
        if (row >= rows) continue;
        const float inv = 1.f / l[i];
        __nv_bfloat16* orow = out + (size_t)(tok0 + row) * o_stride + (size_t)h * D;
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
            const int col = nb * 8 + 2 * (lane & 3);
            *reinterpret_cast<__nv_bfloat162*>(orow + col) = __floats2bfloat162_rn(o[nb][2 * i] * inv, o[nb][2 * i + 1] * inv);
        }
    }
}

template <int D>
int launch_prefill(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                   int table_stride, const int* positions, const int* qo_indptr, const int* tiles, int n_tiles,
                   void* out, int o_stride, int nq, int nkv, int page_size, float scale, int window,
                   cudaStream_t stream) {
    constexpr int S = NsTile<D>::kStride;
    const size_t smem = (size_t)(kTileQ + 4 * kTileKeys) * S * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        NS_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    dim3 grid(n_tiles, nq);
    NS_LAUNCH((attention_prefill_kernel<D>), grid, kPrefillThreads, smem, stream, 
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
        table_stride, positions, qo_indptr, tiles, (__nv_bfloat16*)out, o_stride, nq, nkv, page_size, scale, window);
    NS_CHECK_LAUNCH("ns_attention_prefill");
    return NS_OK;
}

}  // namespace

// tiles: int32 [n_tiles, 2] = (request, offset of the tile's first token among the request's
// tokens of this step, a multiple of 128).  bfloat16 only; head_dim a multiple of 16 up to 128.
NS_API int ns_attention_prefill(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* positions, const int* qo_indptr,
                                const int* tiles, int n_tiles, void* out, int o_stride, int nq, int nkv, int d,
                                int page_size, float scale, int window, cudaStream_t stream) {
    if (n_tiles <= 0) return NS_OK;
    if (d % 16 || d < 16 || d > 128)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill: head_dim=%d (multiples of 16 up to 128)", d);
    if (nkv < 1 || nq % nkv) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill: %d query heads over %d kv heads", nq, nkv);
    if (q_stride % 8 || ((uintptr_t)q % 16) || o_stride % 2)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill: q rows must be 16-byte aligned and out rows 4-byte aligned");
    if (nq > 65535) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill: %d heads exceed the grid's y extent", nq);
#define NS_PREFILL_CASE(DD)                                                                                          \
    case DD:                                                                                                         \
        return launch_prefill<DD>(q, q_stride, k_cache, v_cache, block_table, table_stride, positions, qo_indptr,   \
                                  tiles, n_tiles, out, o_stride, nq, nkv, page_size, scale, window, stream);
    switch (d) {
        NS_PREFILL_CASE(16) NS_PREFILL_CASE(32) NS_PREFILL_CASE(48) NS_PREFILL_CASE(64)
        NS_PREFILL_CASE(80) NS_PREFILL_CASE(96) NS_PREFILL_CASE(112) NS_PREFILL_CASE(128)
    }
#undef NS_PREFILL_CASE
    NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_prefill: head_dim=%d", d);
}
