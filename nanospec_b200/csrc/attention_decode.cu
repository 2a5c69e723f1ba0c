// Decode attention over the paged cache in bfloat16, for every head size in steps of 16 up to 128 and every
// page size (head sizes 64 and 128 with pages of 8 to 64 tokens are served by attention_decode_tma.cu): one
// query token per request, the keys of
// a request split over several thread blocks (split-KV), the query heads that share a kv head
// processed together so that every key and value is read from HBM once per group.
//
// Grid (split, kv head x head tile, token).  A block streams its share of the keys through
// shared memory with cp.async (two or three stages of 64 keys), computes scores and the weighted sum on
// the tensor cores (m16n8k16, the group's heads padded to 16 rows), keeps the softmax in fp32
// (online, base 2), and writes an unnormalised partial result with its running maximum and sum.
// The block that finishes last for a (token, kv head) - found with an atomic counter - merges
// the partials in split order, so the result does not depend on which block came last, and
// resets the counter.  Launch dimensions do not depend on sequence lengths (they are read from
// device memory), which lets a decode step be replayed from a CUDA graph.
//
// Tokens whose request brings more than one token to the step are left to the prefill kernel;
// padding rows (request index < 0) are skipped.
#include "attention_common.cuh"

namespace {

constexpr int kMaxSplits = 16;

// kStages key/value tiles in flight per block: 2 (three blocks per SM) or 3 (two blocks per SM)
template <int D, int kStages>
__global__ void __launch_bounds__(kThreads, kStages == 2 ? 3 : 2)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                        int table_stride, const int* __restrict__ token_req, const int* __restrict__ positions,
                        const int* __restrict__ qo_indptr, __nv_bfloat16* __restrict__ out, int o_stride,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                        const int* __restrict__ rows, int nq, int nkv, int page_size, float scale, int window,
                        int n_splits, int head_tiles) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    using Tile = NsTile<D>;
    constexpr int S = Tile::kStride;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* kv = qs + 16 * S;  // [kStages][k|v][64][S]
    __shared__ int is_last;

    const int split = blockIdx.x, z = blockIdx.z;
    const int n = rows ? rows[z] : z;  // the token this block works for
    const int hk = blockIdx.y / head_tiles, ht = blockIdx.y - hk * head_tiles;
    const int req = token_req[n];
    if (req < 0) return;
    if (qo_indptr[req + 1] - qo_indptr[req] != 1) return;
    const int G = nq / nkv;
    const int h0 = hk * G + ht * 16;
    const int gcount = min(16, G - ht * 16);
    const int pos = positions[n];
    const int kend = pos + 1;
    const int kstart = (window > 0 && kend - window > 0) ? kend - window : 0;
    const int chunk = (((kend - kstart + n_splits - 1) / n_splits + kTileKeys - 1) / kTileKeys) * kTileKeys;
    const int k0 = kstart + split * chunk;
    const int k1 = min(k0 + chunk, kend);
    const int n_tiles = k0 < k1 ? (k1 - k0 + kTileKeys - 1) / kTileKeys : 0;
    const int* bt = block_table + (size_t)req * table_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

    // ---- q of the group's heads (rows beyond the group are zero) and the first tile ----------
    {
        constexpr int kChunks = D / 8;
        const __nv_bfloat16* qrow = q + (size_t)n * q_stride + (size_t)h0 * D;
        for (int c = tid; c < 16 * kChunks; c += kThreads) {
            const int row = c / kChunks, ch = c - row * kChunks;
            const bool valid = row < gcount;
            ns_cp_async16(Tile::at(qs, row, ch * 8), qrow + (valid ? (size_t)row * D + ch * 8 : 0), valid);
        }
    }
    // the first kStages-1 tiles are requested up front; every iteration requests one more
#pragma unroll
    for (int st = 0; st < kStages - 1; ++st) {
        if (st < n_tiles) {
            __nv_bfloat16* kn = kv + (size_t)st * 2 * kTileKeys * S;
            load_kv_tile<D>(kn, kn + kTileKeys * S, k_cache, v_cache, bt, k0 + st * kTileKeys, kstart, k1, hk, nkv, page_size, page_shift);
        }
        ns_cp_async_commit();
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    uint32_t qf[D / 16][4];
    const float sl = scale * kLog2e;
    const int mat = lane >> 3, r8 = lane & 7;

    for (int t = 0; t < n_tiles; ++t) {
        __nv_bfloat16* ks = kv + (size_t)(t % kStages) * 2 * kTileKeys * S;
        __nv_bfloat16* vs = ks + kTileKeys * S;
        __syncthreads();                  // every warp is done with tile t-1: its stage may be refilled
        if (t + kStages - 1 < n_tiles) {
            __nv_bfloat16* kn = kv + (size_t)((t + kStages - 1) % kStages) * 2 * kTileKeys * S;
            load_kv_tile<D>(kn, kn + kTileKeys * S, k_cache, v_cache, bt, k0 + (t + kStages - 1) * kTileKeys, kstart, k1, hk,
                            nkv, page_size, page_shift);
        }
        ns_cp_async_commit();
        ns_cp_async_wait<kStages - 1>();  // tile t has landed; the two after it stay in flight
        __syncthreads();                  // ... for every thread
        if (t == 0) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                ns_ldmatrix_x4(qf[kk], Tile::at(qs, (mat & 1) * 8 + r8, kk * 16 + (mat >> 1) * 8));
        }
        const int kb = k0 + t * kTileKeys + warp * 16;
        if (kb < k1) {
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t kf[4];
                ns_ldmatrix_x4(kf, Tile::at(ks, warp * 16 + (mat >> 1) * 8 + r8, kk * 16 + (mat & 1) * 8));
                ns_mma_bf16(s[0], qf[kk], kf[0], kf[1]);
                ns_mma_bf16(s[1], qf[kk], kf[2], kf[3]);
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int key = kb + nb * 8 + 2 * (lane & 3) + (j & 1);
                    const float v = key < k1 ? s[nb][j] * sl : -INFINITY;
                    s[nb][j] = v;
                    mx[j >> 1] = fmaxf(mx[j >> 1], v);
                }
            float corr[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m[i], mx[i]);  // finite: key kb is valid for every row
                corr[i] = ns_exp2(m[i] - m_new);
                m[i] = m_new;
                l[i] *= corr[i];
            }
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p = ns_exp2(s[nb][j] - m[j >> 1]);
                    s[nb][j] = p;
                    l[j >> 1] += p;
                }
            uint32_t pa[4] = {ns_pack_bf16(s[0][0], s[0][1]), ns_pack_bf16(s[0][2], s[0][3]),
                              ns_pack_bf16(s[1][0], s[1][1]), ns_pack_bf16(s[1][2], s[1][3])};
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
                ns_ldmatrix_x4_trans(vf, Tile::at(vs, warp * 16 + (mat & 1) * 8 + r8, nb2 * 16 + (mat >> 1) * 8));
                ns_mma_bf16(o[2 * nb2], pa, vf[0], vf[1]);
                ns_mma_bf16(o[2 * nb2 + 1], pa, vf[2], vf[3]);
            }
        }
    }
    ns_cp_async_wait<0>();
    __syncthreads();

    // ---- combine the four warps (each saw a quarter of every tile) -----------------------------
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    float* so = reinterpret_cast<float*>(kv);   // [warp][16][D]
    float* sm = so + 4 * 16 * D;                // [warp][16] max, then [warp][16] sum
    {
        const int r0 = lane >> 2;
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb) {
            const int col = nb * 8 + 2 * (lane & 3);
            float* base = so + ((size_t)warp * 16) * D;
            base[(size_t)r0 * D + col] = o[nb][0];
            base[(size_t)r0 * D + col + 1] = o[nb][1];
            base[(size_t)(r0 + 8) * D + col] = o[nb][2];
            base[(size_t)(r0 + 8) * D + col + 1] = o[nb][3];
        }
        if ((lane & 3) == 0) {
            sm[warp * 16 + r0] = m[0];
            sm[warp * 16 + r0 + 8] = m[1];
            sm[64 + warp * 16 + r0] = l[0];
            sm[64 + warp * 16 + r0 + 8] = l[1];
        }
    }
    __syncthreads();
    for (int e = tid; e < gcount * D; e += kThreads) {
        const int row = e / D, col = e - row * D;
        float mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mt = fmaxf(mt, sm[w * 16 + row]);
        float acc = 0.f, lt = 0.f;
        if (mt > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = ns_exp2(sm[w * 16 + row] - mt);
                acc += so[((size_t)w * 16 + row) * D + col] * f;
                lt += sm[64 + w * 16 + row] * f;
            }
        }
        const int h = h0 + row;
        if (n_splits == 1) {
            out[(size_t)n * o_stride + (size_t)h * D + col] = __float2bfloat16_rn(acc / lt);
        } else {
            const size_t slot = ((size_t)z * nq + h) * n_splits + split;
            part_o[slot * D + col] = acc;
            if (col == 0) {
                part_ml[slot * 2] = mt;
                part_ml[slot * 2 + 1] = lt;
            }
        }
    }
    if (n_splits == 1) return;

    // ---- the block that arrives last merges the splits, in split order -------------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* ctr = counters + (size_t)z * gridDim.y + blockIdx.y;
        const int old = atomicAdd(ctr, 1);
        is_last = (old == n_splits - 1);
        if (is_last) *ctr = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int e = tid; e < gcount * D; e += kThreads) {
        const int row = e / D, col = e - row * D;
        const int h = h0 + row;
        const size_t base = ((size_t)z * nq + h) * n_splits;
        // every split's maximum, sum and partial value are requested together, then combined in split order
        float ms[kMaxSplits], ls[kMaxSplits], os[kMaxSplits];
#pragma unroll
        for (int s2 = 0; s2 < kMaxSplits; ++s2) {
            const bool on = s2 < n_splits;
            ms[s2] = on ? __ldcg(part_ml + (base + s2) * 2) : -INFINITY;
            ls[s2] = on ? __ldcg(part_ml + (base + s2) * 2 + 1) : 0.f;
            os[s2] = on ? __ldcg(part_o + (base + s2) * D + col) : 0.f;
        }
        float mt = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < kMaxSplits; ++s2) mt = fmaxf(mt, ms[s2]);
        float acc = 0.f, lt = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < kMaxSplits; ++s2) {
            const float f = ms[s2] == -INFINITY ? 0.f : ns_exp2(ms[s2] - mt);  // an empty split adds nothing
            acc += os[s2] * f;
            lt += ls[s2] * f;
        }
        out[(size_t)n * o_stride + (size_t)h * D + col] = __float2bfloat16_rn(acc / lt);
    }
}

template <int D, int kStages>
int launch_decode_stages(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                  int table_stride, const int* token_req, const int* positions, const int* qo_indptr, void* out,
                  int o_stride, float* part_o, float* part_ml, int* counters, const int* rows, int n_tokens, int nq,
                  int nkv, int page_size, float scale, int window, int n_splits, cudaStream_t stream) {
    constexpr int S = NsTile<D>::kStride;
    const size_t tiles = (size_t)(16 + 2 * kStages * kTileKeys) * S * sizeof(__nv_bfloat16);
    const size_t scratch = (size_t)(4 * 16 * D + 128) * sizeof(float);  // the warps' partial results reuse the k/v stages
    const size_t smem = tiles > 16 * S * sizeof(__nv_bfloat16) + scratch ? tiles : 16 * S * sizeof(__nv_bfloat16) + scratch;
    static bool configured = false;
    if (!configured) {
        NS_CUDA(cudaFuncSetAttribute(attention_decode_kernel<D, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    const int G = nq / nkv, head_tiles = (G + 15) / 16;
    dim3 grid(n_splits, nkv * head_tiles, n_tokens);
    NS_LAUNCH((attention_decode_kernel<D, kStages>), grid, kThreads, smem, stream, 
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
        table_stride, token_req, positions, qo_indptr, (__nv_bfloat16*)out, o_stride, part_o, part_ml, counters, rows, nq,
        nkv, page_size, scale, window, n_splits, head_tiles);
    NS_CHECK_LAUNCH("ns_attention_decode");
    return NS_OK;
}

int g_decode_stages = 3;

template <int D>
int launch_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
                  int table_stride, const int* token_req, const int* positions, const int* qo_indptr, void* out,
                  int o_stride, float* part_o, float* part_ml, int* counters, const int* rows, int n_tokens, int nq,
                  int nkv, int page_size, float scale, int window, int n_splits, cudaStream_t stream) {
    if (g_decode_stages == 2)
        return launch_decode_stages<D, 2>(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions,
                                          qo_indptr, out, o_stride, part_o, part_ml, counters, rows, n_tokens, nq, nkv,
                                          page_size, scale, window, n_splits, stream);
    return launch_decode_stages<D, 3>(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions,
                                      qo_indptr, out, o_stride, part_o, part_ml, counters, rows, n_tokens, nq, nkv,
                                      page_size, scale, window, n_splits, stream);
}

}  // namespace

// Pipeline depth of the decode kernel: 3 stages and two blocks per SM (default) or 2 stages and three.
NS_API int ns_attention_decode_stages(int stages) {
    if (stages != 2 && stages != 3) NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_decode_stages: %d (2 or 3)", stages);
    g_decode_stages = stages;
    return NS_OK;
}

// Scratch sizes for a launch: floats of part_o, floats of part_ml, ints of counters.
NS_API int ns_attention_decode_scratch(int n_tokens, int nq, int nkv, int d, int n_splits, long long* part_o_floats,
                                       long long* part_ml_floats, long long* counter_ints) {
    const int head_tiles = (nq / nkv + 15) / 16;
    *part_o_floats = (long long)n_tokens * nq * n_splits * d;
    *part_ml_floats = (long long)n_tokens * nq * n_splits * 2;
    *counter_ints = (long long)n_tokens * nkv * head_tiles;
    return NS_OK;
}

// bfloat16 only; head_dim a multiple of 16 up to 128.  `counters` must be zero before the first
// launch; every launch leaves it zero again.  `rows` (optional) lists the token rows to work on
// (n_tokens of them); without it the tokens are 0 .. n_tokens-1.
NS_API int ns_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                               const int* block_table, int table_stride, const int* token_req, const int* positions,
                               const int* qo_indptr, void* out, int o_stride, float* part_o, float* part_ml,
                               int* counters, const int* rows, int n_tokens, int nq, int nkv, int d, int page_size,
                               float scale, int window, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (d % 16 || d < 16 || d > 128)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode: head_dim=%d (multiples of 16 up to 128)", d);
    if (nkv < 1 || nq % nkv) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode: %d query heads over %d kv heads", nq, nkv);
    if (n_splits < 1 || n_splits > kMaxSplits) NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_decode: n_splits=%d (1..%d)", n_splits, kMaxSplits);
    if (q_stride % 8 || ((uintptr_t)q % 16)) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode: q rows must be 16-byte aligned");
    if (n_tokens > 65535) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode: %d tokens exceed the grid's z extent", n_tokens);
#define NS_DECODE_CASE(DD)                                                                                             \
    case DD:                                                                                                           \
        return launch_decode<DD>(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions,       \
                                 qo_indptr, out, o_stride, part_o, part_ml, counters, rows, n_tokens, nq, nkv,         \
                                 page_size, scale, window, n_splits, stream);
    switch (d) {
        NS_DECODE_CASE(16) NS_DECODE_CASE(32) NS_DECODE_CASE(48) NS_DECODE_CASE(64)
        NS_DECODE_CASE(80) NS_DECODE_CASE(96) NS_DECODE_CASE(112) NS_DECODE_CASE(128)
    }
#undef NS_DECODE_CASE
    NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode: head_dim=%d", d);
}

// ---------------------------------------------------------------------------------------
// The same kernel for callers that must not allocate: its scratch lives in a fixed array of
// the library image.  Declared and documented in nanospec_b200_noalloc.h.
// ---------------------------------------------------------------------------------------
#include "nanospec_b200_noalloc.h"

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) unsigned char ns_noalloc_scratch[NS_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_noalloc_base[kMaxDevices] = {};  // device address of ns_noalloc_scratch, per device, found on first use

size_t round256(size_t n) { return (n + 255) & ~(size_t)255; }
}  // namespace

NS_API int ns_attention_decode_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                       const int* block_table, int table_stride, const int* token_req,
                                       const int* positions, const int* qo_indptr, void* out, int o_stride,
                                       const int* rows, int n_tokens, int nq, int nkv, int head_dim, int page_size,
                                       float scale, int window, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    // every refusal comes before anything is put on the stream
    if (head_dim % 16 || head_dim < 16 || head_dim > 128)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_noalloc: head_dim=%d (multiples of 16 up to 128)", head_dim);
    if (nkv < 1 || nq < nkv || nq % nkv)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_noalloc: %d query heads over %d kv heads", nq, nkv);
    if (n_splits < 1 || n_splits > kMaxSplits)
        NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_decode_noalloc: n_splits=%d (1..%d)", n_splits, kMaxSplits);
    if (q_stride % 8 || ((uintptr_t)q % 16))
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_noalloc: q rows must be 16-byte aligned");
    if (n_tokens > 65535)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_noalloc: %d tokens exceed the grid's z extent", n_tokens);
    if (n_splits == 1)  // one block sees all of a request's keys: no partial results, no counters, no scratch
        return ns_attention_decode(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions, qo_indptr,
                                   out, o_stride, nullptr, nullptr, nullptr, rows, n_tokens, nq, nkv, head_dim, page_size,
                                   scale, window, 1, stream);
    long long o_floats, ml_floats, ctr_ints;
    ns_attention_decode_scratch(n_tokens, nq, nkv, head_dim, n_splits, &o_floats, &ml_floats, &ctr_ints);
    const size_t ctr_bytes = round256((size_t)ctr_ints * sizeof(int));
    const size_t ml_bytes = round256((size_t)ml_floats * sizeof(float));
    const size_t o_bytes = round256((size_t)o_floats * sizeof(float));
    const size_t need = ctr_bytes + ml_bytes + o_bytes;
    if (need > NS_NOALLOC_SCRATCH_BYTES)
        NS_FAIL(NS_ERR_UNSUPPORTED,
                "ns_attention_decode_noalloc: %d tokens x %d heads x %d splits x head_dim %d need %zu bytes of scratch; "
                "the built-in array holds %u (use fewer splits or tokens, or ns_attention_decode with your own scratch)",
                n_tokens, nq, n_splits, head_dim, need, NS_NOALLOC_SCRATCH_BYTES);
    int dev = 0;
    NS_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_decode_noalloc: device %d", dev);
    if (g_noalloc_base[dev] == nullptr) {
        // set-up, once per device, with that device current: the array's address on this device
        void* p = nullptr;
        NS_CUDA(cudaGetSymbolAddress(&p, ns_noalloc_scratch));
        g_noalloc_base[dev] = p;
    }
    unsigned char* base = static_cast<unsigned char*>(g_noalloc_base[dev]);
    int* counters = reinterpret_cast<int*>(base);
    float* part_ml = reinterpret_cast<float*>(base + ctr_bytes);
    float* part_o = reinterpret_cast<float*>(base + ctr_bytes + ml_bytes);
    // the array keeps whatever the last call left: the arrival counters must start at zero
    NS_CUDA(cudaMemsetAsync(counters, 0, ctr_bytes, stream));
    return ns_attention_decode(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions, qo_indptr,
                               out, o_stride, part_o, part_ml, counters, rows, n_tokens, nq, nkv, head_dim, page_size,
                               scale, window, n_splits, stream);
}
