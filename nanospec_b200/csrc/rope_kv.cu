// Rotary position encoding of q and k fused with the write of k and v into the paged cache.
//
// Per token: angle[j] = float(position) * inv_freq[j] (fp32, accurate sincosf), pairs are
// (x[j], x[j + d/2]) ("rotate half"): out[j] = x[j] cos - x[j+d/2] sin,
// out[j+d/2] = x[j+d/2] cos + x[j] sin.  q is rotated in place in the packed projection
// [q | k | v]; the rotated k and the untouched v go to the cache slot that the request's
// block table gives for the token's position:
//   page = block_table[request, position / page_size],  cache[page, kv head, position % page_size, :].
// A token whose request index is negative is a padding row and is skipped.
#include "common.cuh"

namespace {

// One block per (token, head): heads 0..nq-1 are q (rotated in place), nq..nq+nkv-1 are k (rotated
// into the cache), the last nkv are v (copied into the cache).  Thread j owns the pair (j, j + d/2).
template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_req,
                     const int* __restrict__ block_table, int table_stride, const float* __restrict__ inv_freq,
                     T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int nq, int nkv, int d,
                     int rot_pairs, int write_kv) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    // The step's description, the block table and the angles do not come from the previous kernel: they
    // are read and computed before this kernel waits for it; only the projection itself comes after.
    const int n = blockIdx.x, hh = blockIdx.y;
    const int req = token_req[n];
    // a block with nothing to do still waits: a grid whose blocks all left early would complete while its
    // predecessor runs, and its successor's wait would then cover this grid only
    if (req < 0) { ns_pdl_wait(); return; }
    const bool is_q = hh < nq, is_v = hh >= nq + nkv;
    if (!is_q && !write_kv) { ns_pdl_wait(); return; }
    const int pos = positions[n];
    const int half = d / 2;
    T* x = qkv + (size_t)n * (nq + 2 * nkv) * d + (size_t)hh * d;
    T* dst = x;
    if (!is_q) {
        const int page = block_table[(size_t)req * table_stride + pos / page_size];
        const int hk = is_v ? hh - nq - nkv : hh - nq;
        // cache[page, kv head, offset, :]
        dst = (is_v ? v_cache : k_cache) + (((size_t)page * nkv + hk) * page_size + pos % page_size) * d;
    }
    const int j0 = threadIdx.x;  // a block of 128 threads covers head sizes up to 256 in one pass
    float s0 = 0.f, c0 = 1.f;
    if (!is_v && j0 < rot_pairs && j0 < half) sincosf((float)pos * inv_freq[j0], &s0, &c0);
    ns_pdl_wait();               // everything below sees the previous kernel's results
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float x1 = ns_ld(x, j), x2 = ns_ld(x, j + half);
        float o1 = x1, o2 = x2;
        if (!is_v && j < rot_pairs) {
            float s = s0, c = c0;
            if (j != j0) sincosf((float)pos * inv_freq[j], &s, &c);
            // spelled out so that both kernels of this file round alike
            o1 = __fmaf_rn(x1, c, -__fmul_rn(x2, s));
            o2 = __fmaf_rn(x2, c, __fmul_rn(x1, s));
        }
        ns_st(dst, j, o1);
        ns_st(dst, j + half, o2);
    }
}

// The same work with one block per token (all heads), for steps with many tokens: a block per
// (token, head) would then be bound by the rate at which blocks can be scheduled.  cos and sin of
// the token's angles are computed once and shared through shared memory.
template <typename T, bool kVec>
__global__ void __launch_bounds__(256)
rope_kv_write_token_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_req,
                           const int* __restrict__ block_table, int table_stride, const float* __restrict__ inv_freq,
                           T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int nq, int nkv, int d,
                           int rot_pairs, int write_kv) {
    ns_pdl_launch_dependents();
    // The token's request, position, page and angles do not come from the previous kernel (the step's
    // description and the block table are written before the step's first kernel): they are read and
    // computed before this kernel waits for it; only the projection itself comes after.
    extern __shared__ float cs[];  // [rot_pairs] cos, then [rot_pairs] sin
    const int n = blockIdx.x;
    const int req = token_req[n];
    if (req < 0) { ns_pdl_wait(); return; }  // (see rope_kv_write_kernel)
    const int pos = positions[n];
    const int half = d / 2;
    for (int j = threadIdx.x; j < rot_pairs; j += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        cs[j] = c;
        cs[rot_pairs + j] = s;
    }
    T* row = qkv + (size_t)n * (nq + 2 * nkv) * d;
    size_t base = 0;
    if (write_kv) {
        const int page = block_table[(size_t)req * table_stride + pos / page_size];
        base = ((size_t)page * nkv * page_size + pos % page_size) * d;  // cache[page, 0, offset, :]
    }
    __syncthreads();
    ns_pdl_wait();
    const size_t head_stride = (size_t)page_size * d;                   // from one kv head to the next
    const int rot_heads = write_kv ? nq + nkv : nq;
    if (kVec) {
        // half a head is a multiple of 8 elements and every row is 16-byte aligned: 8 pairs per thread and turn
        const int per_head = half / 8;
        for (int i = threadIdx.x; i < rot_heads * per_head; i += blockDim.x) {
            const int h = i / per_head, j = (i - h * per_head) * 8;
            T* x = row + (size_t)h * d;
            float x1[8], x2[8], o1[8], o2[8];
            ld8(x + j, x1);
            ld8(x + j + half, x2);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                o1[u] = x1[u];
                o2[u] = x2[u];
                if (j + u < rot_pairs) {
                    const float c = cs[j + u], s = cs[rot_pairs + j + u];
                    o1[u] = __fmaf_rn(x1[u], c, -__fmul_rn(x2[u], s));
                    o2[u] = __fmaf_rn(x2[u], c, __fmul_rn(x1[u], s));
                }
            }
            T* dst = h < nq ? x : k_cache + base + (size_t)(h - nq) * head_stride;
            st8(dst + j, o1);
            st8(dst + j + half, o2);
        }
        if (write_kv) {
            const T* v = row + (size_t)(nq + nkv) * d;
            const int per_v = d / 8;
            for (int i = threadIdx.x; i < nkv * per_v; i += blockDim.x) {
                const int hk = i / per_v, e = (i - hk * per_v) * 8;
                float t[8];
                ld8(v + (size_t)hk * d + e, t);
                st8(v_cache + base + (size_t)hk * head_stride + e, t);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < rot_heads * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        T* x = row + (size_t)h * d;
        const float x1 = ns_ld(x, j), x2 = ns_ld(x, j + half);
        float o1 = x1, o2 = x2;
        if (j < rot_pairs) {
            const float c = cs[j], s = cs[rot_pairs + j];
            o1 = __fmaf_rn(x1, c, -__fmul_rn(x2, s));
            o2 = __fmaf_rn(x2, c, __fmul_rn(x1, s));
        }
        T* dst = h < nq ? x : k_cache + base + (size_t)(h - nq) * head_stride;
        ns_st(dst, j, o1);
        ns_st(dst, j + half, o2);
    }
    if (write_kv) {
        const T* v = row + (size_t)(nq + nkv) * d;
        for (int i = threadIdx.x; i < nkv * d; i += blockDim.x) {
            const int hk = i / d, e = i - hk * d;
            v_cache[base + (size_t)hk * head_stride + e] = v[i];
        }
    }
}

int g_token_kernel_from = 48;  // measured in a decode step of 64 tokens: 4.80 ms with a block per token, 5.02 ms with one per (token, head)

}  // namespace

// Steps with at least this many tokens take the kernel with one block per token (default 48).
NS_API int ns_rope_token_kernel_from(int n_tokens) {
    if (n_tokens < 1) NS_FAIL(NS_ERR_ARGUMENT, "ns_rope_token_kernel_from: %d", n_tokens);
    g_token_kernel_from = n_tokens;
    return NS_OK;
}

// rot_pairs = number of (j, j + d/2) pairs that are rotated (d/2 for full rotary).
NS_API int ns_rope_kv_write(void* qkv, const int* positions, const int* token_req, const int* block_table,
                            int table_stride, const float* inv_freq, void* k_cache, void* v_cache, int page_size,
                            int nq, int nkv, int d, int rot_pairs, int n_tokens, int write_kv, int dtype,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (d % 2 || rot_pairs > d / 2 || rot_pairs < 0)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_rope_kv_write: head_dim=%d rot_pairs=%d (head_dim must be even, pairs <= head_dim/2)", d, rot_pairs);
    if (nq + 2 * nkv > 65535) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_rope_kv_write: %d heads exceed the grid", nq + 2 * nkv);
    if (n_tokens >= g_token_kernel_from && 2 * (size_t)rot_pairs * sizeof(float) <= 48 * 1024) {
        const size_t smem = 2 * (size_t)rot_pairs * sizeof(float);
        // 16-byte accesses when half a head is a multiple of 8 elements and the tensors are 16-byte aligned
        // (rows of qkv and of the cache are then aligned too); the arithmetic is the same either way
        const bool vec = d % 16 == 0 && (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0) &&
                         (dtype == NS_F32 || dtype == NS_BF16);
        if (dtype == NS_F32 && vec)
            NS_LAUNCH((rope_kv_write_token_kernel<float, true>), n_tokens, 256, smem, stream, (float*)qkv, positions, token_req,
                      block_table, table_stride, inv_freq, (float*)k_cache, (float*)v_cache, page_size, nq, nkv, d,
                      rot_pairs, write_kv);
        else if (dtype == NS_BF16 && vec)
            NS_LAUNCH((rope_kv_write_token_kernel<__nv_bfloat16, true>), n_tokens, 256, smem, stream, (__nv_bfloat16*)qkv,
                      positions, token_req, block_table, table_stride, inv_freq, (__nv_bfloat16*)k_cache,
                      (__nv_bfloat16*)v_cache, page_size, nq, nkv, d, rot_pairs, write_kv);
        else if (dtype == NS_F32)
            NS_LAUNCH((rope_kv_write_token_kernel<float, false>), n_tokens, 256, smem, stream, (float*)qkv, positions, token_req,
                      block_table, table_stride, inv_freq, (float*)k_cache, (float*)v_cache, page_size, nq, nkv, d,
                      rot_pairs, write_kv);
        else if (dtype == NS_BF16)
            NS_LAUNCH((rope_kv_write_token_kernel<__nv_bfloat16, false>), n_tokens, 256, smem, stream, (__nv_bfloat16*)qkv,
                      positions, token_req, block_table, table_stride, inv_freq, (__nv_bfloat16*)k_cache,
                      (__nv_bfloat16*)v_cache, page_size, nq, nkv, d, rot_pairs, write_kv);
        else
            NS_FAIL(NS_ERR_ARGUMENT, "ns_rope_kv_write: unknown dtype %d", dtype);
        NS_CHECK_LAUNCH("ns_rope_kv_write");
        return NS_OK;
    }
    const dim3 grid(n_tokens, nq + 2 * nkv);
    const int threads = d / 2 <= 32 ? 32 : (d / 2 <= 64 ? 64 : 128);
    if (dtype == NS_F32)
        NS_LAUNCH((rope_kv_write_kernel<float>), grid, threads, 0, stream, 
            (float*)qkv, positions, token_req, block_table, table_stride, inv_freq, (float*)k_cache, (float*)v_cache,
            page_size, nq, nkv, d, rot_pairs, write_kv);
    else if (dtype == NS_BF16)
        NS_LAUNCH((rope_kv_write_kernel<__nv_bfloat16>), grid, threads, 0, stream, 
            (__nv_bfloat16*)qkv, positions, token_req, block_table, table_stride, inv_freq, (__nv_bfloat16*)k_cache,
            (__nv_bfloat16*)v_cache, page_size, nq, nkv, d, rot_pairs, write_kv);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_rope_kv_write: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_rope_kv_write");
    return NS_OK;
}
