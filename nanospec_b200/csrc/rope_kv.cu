// Rotary position encoding of q and k fused with the write of k and v into the paged cache.
//
// Per token: angle[j] = float(position) * inv_freq[j] (fp32, accurate sincosf), pairs are
// (x[j], x[j + d/2]) ("rotate half"): out[j] = x[j] cos - x[j+d/2] sin,
// out[j+d/2] = x[j+d/2] cos + x[j] sin.  q is rotated in place in the packed projection
// [q | k | v]; the rotated k and the untouched v go to the cache slot that the request's
// block table gives for the token's position:
//   page = block_table[request, position / page_size],  slot = page * page_size + position % page_size.
// A token whose request index is negative is a padding row and is skipped.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_req,
                     const int* __restrict__ block_table, int table_stride, const float* __restrict__ inv_freq,
                     T* __restrict__ k_cache, T* __restrict__ v_cache, int page_size, int nq, int nkv, int d,
                     int rot_pairs, int write_kv) {
    extern __shared__ float cs[];  // [rot_pairs] cos, then [rot_pairs] sin
    const int n = blockIdx.x;
    const int req = token_req[n];
    if (req < 0) return;
    const int pos = positions[n];
    const int half = d / 2;
    for (int j = threadIdx.x; j < rot_pairs; j += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        cs[j] = c;
        cs[rot_pairs + j] = s;
    }
    __syncthreads();

    const int row_width = (nq + 2 * nkv) * d;
    T* row = qkv + (size_t)n * row_width;
    size_t slot = 0;
    if (write_kv) {
        const int page = block_table[(size_t)req * table_stride + pos / page_size];
        slot = (size_t)page * page_size + pos % page_size;
    }
    T* kdst = k_cache + slot * nkv * d;
    T* vdst = v_cache + slot * nkv * d;

    // rotation of q heads (in place) and k heads (to the cache)
    const int rot_heads = nq + nkv;
    for (int i = threadIdx.x; i < rot_heads * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        T* x = row + (size_t)h * d;
        const float x1 = ns_ld(x, j), x2 = ns_ld(x, j + half);
        float o1 = x1, o2 = x2;
        if (j < rot_pairs) {
            const float c = cs[j], s = cs[rot_pairs + j];
            o1 = x1 * c - x2 * s;
            o2 = x2 * c + x1 * s;
        }
        if (h < nq) {
            ns_st(x, j, o1);
            ns_st(x, j + half, o2);
        } else if (write_kv) {
            T* kd = kdst + (size_t)(h - nq) * d;
            ns_st(kd, j, o1);
            ns_st(kd, j + half, o2);
        }
    }
    if (write_kv) {
        const T* v = row + (size_t)(nq + nkv) * d;
        for (int i = threadIdx.x; i < nkv * d; i += blockDim.x) vdst[i] = v[i];
    }
}

}  // namespace

// rot_pairs = number of (j, j + d/2) pairs that are rotated (d/2 for full rotary).
NS_API int ns_rope_kv_write(void* qkv, const int* positions, const int* token_req, const int* block_table,
                            int table_stride, const float* inv_freq, void* k_cache, void* v_cache, int page_size,
                            int nq, int nkv, int d, int rot_pairs, int n_tokens, int write_kv, int dtype,
                            cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    if (d % 2 || rot_pairs > d / 2 || rot_pairs < 0)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_rope_kv_write: head_dim=%d rot_pairs=%d (head_dim must be even, pairs <= head_dim/2)", d, rot_pairs);
    const size_t smem = 2 * (size_t)rot_pairs * sizeof(float);
    if (smem > 48 * 1024) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_rope_kv_write: head_dim=%d is too large", d);
    if (dtype == NS_F32)
        rope_kv_write_kernel<float><<<n_tokens, 128, smem, stream>>>(
            (float*)qkv, positions, token_req, block_table, table_stride, inv_freq, (float*)k_cache, (float*)v_cache,
            page_size, nq, nkv, d, rot_pairs, write_kv);
    else if (dtype == NS_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<n_tokens, 128, smem, stream>>>(
            (__nv_bfloat16*)qkv, positions, token_req, block_table, table_stride, inv_freq, (__nv_bfloat16*)k_cache,
            (__nv_bfloat16*)v_cache, page_size, nq, nkv, d, rot_pairs, write_kv);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_rope_kv_write: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_rope_kv_write");
    return NS_OK;
}
