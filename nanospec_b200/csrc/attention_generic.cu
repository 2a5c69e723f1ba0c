// Attention over the paged cache, one warp per (token, query head), any head size up to 256.
//
// This is the exact kernel: every score, the softmax and the weighted sum are fp32 with
// accurate expf, and the keys of one query are always visited in the same order (ascending
// from the first key it may see, 32 at a time), so a query's output does not depend on how
// the batch was cut into steps or on what else runs beside it.  The true 32-bit path uses
// it for every step; the bfloat16 path uses it for sizes that the tensor-core kernels refuse.
//
// A query at position p of request r sees the keys at positions max(0, p - window + 1) .. p
// of the same request (window == 0: all of 0 .. p).  Keys and values are read from
// cache[page, kv_head, offset, :] with page = block_table[r, position / page_size]; the
// step's own keys have been written before this kernel runs.  kv_head = q_head / (nq / nkv).
#include "common.cuh"

namespace {

constexpr int kWarpsPerBlock = 4;

template <typename T, int DPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attention_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                         const T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ token_req, const int* __restrict__ positions, T* __restrict__ out,
                         int o_stride, int n_tokens, int nq, int nkv, int d, int page_size, float scale, int window) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    extern __shared__ float qsm[];
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long w = (long long)blockIdx.x * kWarpsPerBlock + wib;
    if (w >= (long long)n_tokens * nq) return;
    const int n = (int)(w / nq), h = (int)(w % nq);
    T* o = out + (size_t)n * o_stride + (size_t)h * d;
    const int req = token_req[n];
    if (req < 0) return;
    const int pos = positions[n];
    const int hk = h / (nq / nkv);
    const int kend = pos + 1;
    const int kstart = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    float* qs = qsm + wib * d;
    const T* qrow = q + (size_t)n * q_stride + (size_t)h * d;
    for (int e = lane; e < d; e += 32) qs[e] = ns_ld(qrow, e);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    const int* bt = block_table + (size_t)req * table_stride;

    for (int kb = kstart; kb < kend; kb += 32) {
        const int key = kb + lane;
        const bool valid = key < kend;
        unsigned slot = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[key / page_size];
            // row of cache[page, kv head, offset, :]
            slot = ((unsigned)page * (unsigned)nkv + (unsigned)hk) * (unsigned)page_size + (unsigned)(key % page_size);
            const T* kr = k_cache + (size_t)slot * d;
            float dot = 0.f;
            for (int e = 0; e < d; ++e) dot = fmaf(qs[e], ns_ld(kr, e), dot);
            s = dot * scale;
        }
        const float m_new = fmaxf(m, ns_warp_max(s));
        const float corr = expf(m - m_new);  // first chunk: exp(-inf) = 0
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + ns_warp_sum(p);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[i] *= corr;
        const int cnt = min(32, kend - kb);
        for (int j = 0; j < cnt; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const unsigned sj = __shfl_sync(0xffffffffu, slot, j);
            const T* vr = v_cache + (size_t)sj * d;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int e = lane + 32 * i;
                if (e < d) acc[i] = fmaf(pj, ns_ld(vr, e), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
        const int e = lane + 32 * i;
        if (e < d) ns_st(o, e, acc[i] * inv);
    }
}

template <typename T>
int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache, const int* block_table,
           int table_stride, const int* token_req, const int* positions, void* out, int o_stride, int n_tokens, int nq,
           int nkv, int d, int page_size, float scale, int window, cudaStream_t stream) {
    const long long warps = (long long)n_tokens * nq;
    const unsigned blocks = (unsigned)((warps + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const size_t smem = (size_t)kWarpsPerBlock * d * sizeof(float);
    const int dpl = (d + 31) / 32;
#define NS_ATTN_CASE(D)                                                                                              \
    case D:                                                                                                          \
        NS_LAUNCH((attention_generic_kernel<T, D>), blocks, kWarpsPerBlock * 32, smem, stream,                                \
            (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, block_table, table_stride, token_req,       \
            positions, (T*)out, o_stride, n_tokens, nq, nkv, d, page_size, scale, window);                           \
        break;
    switch (dpl) {
        NS_ATTN_CASE(1) NS_ATTN_CASE(2) NS_ATTN_CASE(3) NS_ATTN_CASE(4)
        NS_ATTN_CASE(5) NS_ATTN_CASE(6) NS_ATTN_CASE(7) NS_ATTN_CASE(8)
    }
#undef NS_ATTN_CASE
    NS_CHECK_LAUNCH("ns_attention_generic");
    return NS_OK;
}

}  // namespace

NS_API int ns_attention_generic(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* token_req, const int* positions,
                                void* out, int o_stride, int n_tokens, int nq, int nkv, int d, int page_size,
                                float scale, int window, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (d < 1 || d > 256) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_generic: head_dim=%d is outside 1..256", d);
    if (nkv < 1 || nq % nkv) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_attention_generic: %d query heads over %d kv heads", nq, nkv);
    if (dtype == NS_F32)
        return launch<float>(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions, out,
                             o_stride, n_tokens, nq, nkv, d, page_size, scale, window, stream);
    if (dtype == NS_BF16)
        return launch<__nv_bfloat16>(q, q_stride, k_cache, v_cache, block_table, table_stride, token_req, positions,
                                     out, o_stride, n_tokens, nq, nkv, d, page_size, scale, window, stream);
    NS_FAIL(NS_ERR_ARGUMENT, "ns_attention_generic: unknown dtype %d", dtype);
}
