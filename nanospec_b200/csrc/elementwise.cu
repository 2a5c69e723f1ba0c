// Embedding gather, RMSNorm with the residual sum fused in, and the SwiGLU gate.
//
// The residual stream is float in every precision mode: the sum of branch outputs is kept
// in 32-bit and only the normalised activations that feed a matrix product are rounded to
// the compute type.
#include "common.cuh"

thread_local char ns_error_text[512] = "";
NS_API const char* ns_last_error() { return ns_error_text; }

int ns_pdl_enabled = 1;
// 1 (default): kernels are launched so that they may overlap the tail of their predecessor
// (programmatic dependent launch); 0: plain stream order.
NS_API int ns_set_pdl(int enabled) {
    ns_pdl_enabled = enabled ? 1 : 0;
    return NS_OK;
}

// ---------------------------------------------------------------------------------------
// embedding: out[n, :] = float(table[ids[n], :]); a negative id (padding row) gives zeros
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                             int hidden, int vocab) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    const int n = blockIdx.x;
    const int id = ids[n];
    float* o = out + (size_t)n * hidden;
    if (id < 0 || id >= vocab) {
        for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) o[h] = ns_ld(row, h);
}

NS_API int ns_embed(const void* table, const int* ids, float* out, int n_tokens, int hidden, int vocab, int dtype,
                    cudaStream_t stream) {
    if (n_tokens <= 0) return NS_OK;
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    if (dtype == NS_F32)
        NS_LAUNCH((embed_kernel<float>), n_tokens, threads, 0, stream, (const float*)table, ids, out, hidden, vocab);
    else if (dtype == NS_BF16)
        NS_LAUNCH((embed_kernel<__nv_bfloat16>), n_tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, hidden, vocab);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_embed: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_embed");
    return NS_OK;
}

// ---------------------------------------------------------------------------------------
// token ids that an earlier step sampled and the host has not seen yet: ids[dst_rows[i]] = src[src_rows[i]]
// ---------------------------------------------------------------------------------------
__global__ void take_ids_kernel(int* __restrict__ ids, const int* __restrict__ dst_rows, const int* __restrict__ src,
                                const int* __restrict__ src_rows, int n) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ids[dst_rows[i]] = src[src_rows[i]];
}

NS_API int ns_take_ids(int* ids, const int* dst_rows, const int* src, const int* src_rows, int n, cudaStream_t stream) {
    if (n <= 0) return NS_OK;
    NS_LAUNCH(take_ids_kernel, (n + 127) / 128, 128, 0, stream, ids, dst_rows, src, src_rows, n);
    NS_CHECK_LAUNCH("ns_take_ids");
    return NS_OK;
}

// ---------------------------------------------------------------------------------------
// RMSNorm over the residual stream, with the pending branch output added first:
//   r = resid[row] + branch[row]        (branch may be absent)
//   resid[row] = r                      (when write_resid)
//   out[j]  = r * rsqrt(mean(r^2) + eps) * gain          all in float, rounded once to T
// `rows` (optional) selects the input rows: output row j reads input row rows[j]; then the
// residual is not written back (used for the final norm at the wanted positions).
// ---------------------------------------------------------------------------------------
template <typename T, int THREADS, int PER_THREAD>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ branch, const float* __restrict__ gain,
                   T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps, int write_resid) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    __shared__ float scratch[32];
    const int j = blockIdx.x;
    const int row = rows ? rows[j] : j;
    float* r = resid + (size_t)row * hidden;
    const T* b = branch ? branch + (size_t)row * hidden : nullptr;
    T* o = out + (size_t)j * hidden;

    float v[PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int h = threadIdx.x + i * THREADS;
        float x = 0.f;
        if (h < hidden) {
            x = r[h];
            if (b) x += ns_ld(b, h);
            if (write_resid && b) r[h] = x;
        }
        v[i] = x;
        ss += x * x;
    }
    // elements beyond PER_THREAD * THREADS (very wide rows) are handled from memory
    for (int h = threadIdx.x + PER_THREAD * THREADS; h < hidden; h += THREADS) {
        float x = r[h];
        if (b) x += ns_ld(b, h);
        if (write_resid && b) r[h] = x;
        ss += x * x;
    }
    const float total = ns_block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < PER_THREAD; ++i) {
        const int h = threadIdx.x + i * THREADS;
        if (h < hidden) ns_st(o, h, v[i] * inv * gain[h]);
    }
    for (int h = threadIdx.x + PER_THREAD * THREADS; h < hidden; h += THREADS) {
        float x = r[h];
        if (b && !write_resid) x += ns_ld(b, h);
        ns_st(o, h, x * inv * gain[h]);
    }
}

// Vector variant for widths that are a multiple of 8 with 16-byte aligned rows: every thread owns
// CHUNKS groups of 8 consecutive elements, read and written with 16-byte accesses.
template <typename T, int THREADS, int CHUNKS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ branch, const float* __restrict__ gain,
                       T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps, int write_resid) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    __shared__ float scratch[32];
    // the gain is a weight: it is fetched while the previous kernel is still running
    float g[CHUNKS][8];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int h = (threadIdx.x + c * THREADS) * 8;
        if (h < hidden) ld8(gain + h, g[c]);
    }
    ns_pdl_wait();               // everything below sees the previous kernel's results
    const int j = blockIdx.x;
    const int row = rows ? rows[j] : j;
    float* r = resid + (size_t)row * hidden;
    const T* b = branch ? branch + (size_t)row * hidden : nullptr;
    T* o = out + (size_t)j * hidden;
    float v[CHUNKS][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int h = (threadIdx.x + c * THREADS) * 8;
        if (h < hidden) {
            ld8(r + h, v[c]);
            if (b) {
                float t[8];
                ld8(b + h, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[c][i] += t[i];
                if (write_resid) st8(r + h, v[c]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += v[c][i] * v[c][i];
        }
    }
    const float inv = rsqrtf(ns_block_sum(ss, scratch) / (float)hidden + eps);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int h = (threadIdx.x + c * THREADS) * 8;
        if (h < hidden) {
            float y[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = v[c][i] * inv * g[c][i];
            st8(o + h, y);
        }
    }
}

template <typename T>
static int launch_add_rmsnorm(float* resid, const void* branch, const float* gain, void* out, const int* rows,
                              int n_rows, int hidden, float eps, int write_resid, cudaStream_t stream) {
    const T* b = (const T*)branch;
    T* o = (T*)out;
    const bool aligned = hidden % 8 == 0 && (((uintptr_t)resid | (uintptr_t)branch | (uintptr_t)gain | (uintptr_t)out) % 16 == 0);
    if (aligned && hidden >= 1024 && hidden <= 16384) {
        // the sum of squares runs over the same elements in another grouping than the scalar kernel;
        // which kernel runs depends on the width and alignment only, never on the batch
        if (hidden <= 2048)
            NS_LAUNCH((add_rmsnorm_vec_kernel<T, 128, 2>), n_rows, 128, 0, stream, resid, b, gain, o, rows, hidden, eps, write_resid);
        else if (hidden <= 4096)
            NS_LAUNCH((add_rmsnorm_vec_kernel<T, 256, 2>), n_rows, 256, 0, stream, resid, b, gain, o, rows, hidden, eps, write_resid);
        else if (hidden <= 8192)
            NS_LAUNCH((add_rmsnorm_vec_kernel<T, 512, 2>), n_rows, 512, 0, stream, resid, b, gain, o, rows, hidden, eps, write_resid);
        else
            NS_LAUNCH((add_rmsnorm_vec_kernel<T, 1024, 2>), n_rows, 1024, 0, stream, resid, b, gain, o, rows, hidden, eps, write_resid);
        NS_CHECK_LAUNCH("ns_add_rmsnorm");
        return NS_OK;
    }
    if (hidden <= 256)
        NS_LAUNCH((add_rmsnorm_kernel<T, 64, 4>), n_rows, 64, 0, stream, resid, b, gain, o, rows, hidden, eps, write_resid);
    else if (hidden <= 1024)
        NS_LAUNCH((add_rmsnorm_kernel<T, 128, 8>), n_rows, 128, 0, stream, resid, b, gain, o, rows, hidden, eps, write_resid);
    else if (hidden <= 4096)
        NS_LAUNCH((add_rmsnorm_kernel<T, 512, 8>), n_rows, 512, 0, stream, resid, b, gain, o, rows, hidden, eps, write_resid);
    else
        NS_LAUNCH((add_rmsnorm_kernel<T, 1024, 8>), n_rows, 1024, 0, stream, resid, b, gain, o, rows, hidden, eps, write_resid);
    NS_CHECK_LAUNCH("ns_add_rmsnorm");
    return NS_OK;
}

NS_API int ns_add_rmsnorm(float* resid, const void* branch, const float* gain, void* out, const int* rows, int n_rows,
                          int hidden, float eps, int write_resid, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return NS_OK;
    if (hidden <= 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_add_rmsnorm: hidden=%d", hidden);
    if (rows && write_resid) NS_FAIL(NS_ERR_ARGUMENT, "ns_add_rmsnorm: a row selection cannot write the residual back");
    if (dtype == NS_F32)
        return launch_add_rmsnorm<float>(resid, branch, gain, out, rows, n_rows, hidden, eps, write_resid, stream);
    if (dtype == NS_BF16)
        return launch_add_rmsnorm<__nv_bfloat16>(resid, branch, gain, out, rows, n_rows, hidden, eps, write_resid, stream);
    NS_FAIL(NS_ERR_ARGUMENT, "ns_add_rmsnorm: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------
// residual sum alone: resid[row] += branch[row]  (used when no norm follows)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ resid, const T* __restrict__ branch, size_t n) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) resid[i] += ns_ld(branch, i);
}

NS_API int ns_residual_add(float* resid, const void* branch, int n_rows, int hidden, int dtype, cudaStream_t stream) {
    const size_t n = (size_t)n_rows * hidden;
    if (n == 0) return NS_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == NS_F32)
        NS_LAUNCH((residual_add_kernel<float>), blocks, 256, 0, stream, resid, (const float*)branch, n);
    else if (dtype == NS_BF16)
        NS_LAUNCH((residual_add_kernel<__nv_bfloat16>), blocks, 256, 0, stream, resid, (const __nv_bfloat16*)branch, n);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_residual_add: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_residual_add");
    return NS_OK;
}

// ---------------------------------------------------------------------------------------
// SwiGLU gate on the packed [gate | up] projection:
//   out[n, j] = silu(gu[n, j]) * gu[n, inter + j],  silu(a) = a / (1 + exp(-a)),  in float
// ---------------------------------------------------------------------------------------
// silu(g) * u.  The float kernels use the accurate exponential and division; the bfloat16 ones the
// hardware approximations (about 2 ulp in float, far below the rounding of the result).
template <typename T>
__device__ __forceinline__ float silu_mul(float g, float u) { return (g / (1.f + expf(-g))) * u; }
template <>
__device__ __forceinline__ float silu_mul<__nv_bfloat16>(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, int block, size_t total) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t n = i / inter;
    const int j = (int)(i - n * inter);
    // block == 0: [gate | up]; otherwise gate and up alternate in runs of `block` features
    const size_t gi = block ? (size_t)(j / block) * 2 * block + j % block : (size_t)j;
    const float g = ns_ld(gu, n * 2 * (size_t)inter + gi);
    const float u = ns_ld(gu, n * 2 * (size_t)inter + gi + (block ? block : inter));
    ns_st(out, i, silu_mul<T>(g, u));
}

template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, int block, size_t total8) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const int per_row = inter / 8;
    const size_t n = i / per_row;
    const int j = (int)(i - n * per_row) * 8;
    float g[8], u[8], y[8];
    const size_t gi = block ? (size_t)(j / block) * 2 * block + j % block : (size_t)j;  // block is a multiple of 8
    ld8(gu + n * 2 * (size_t)inter + gi, g);
    ld8(gu + n * 2 * (size_t)inter + gi + (block ? block : inter), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) y[k] = silu_mul<T>(g[k], u[k]);
    st8(out + n * (size_t)inter + j, y);
}

// out[n, j] = silu(g) * u with g, u = gate_up[n, j], gate_up[n, inter + j] (block == 0), or, when gate and up
// alternate in runs of `block` features (a multiple of 8 that divides inter), gate_up[n, (j / block) * 2 * block +
// j % block] and the element `block` further.
NS_API int ns_swiglu(const void* gate_up, void* out, int n_rows, int inter, int block, int dtype, cudaStream_t stream) {
    const size_t total = (size_t)n_rows * inter;
    if (total == 0) return NS_OK;
    if (block < 0 || (block && (block % 8 || inter % block)))
        NS_FAIL(NS_ERR_ARGUMENT, "ns_swiglu: block=%d must be 0 or a multiple of 8 that divides %d", block, inter);
    if (inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) % 16 == 0)) {
        const size_t total8 = total / 8;
        const unsigned vblocks = (unsigned)((total8 + 255) / 256);
        if (dtype == NS_F32)
            NS_LAUNCH((swiglu_vec_kernel<float>), vblocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter, block, total8);
        else if (dtype == NS_BF16)
            NS_LAUNCH((swiglu_vec_kernel<__nv_bfloat16>), vblocks, 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block, total8);
        else
            NS_FAIL(NS_ERR_ARGUMENT, "ns_swiglu: unknown dtype %d", dtype);
        NS_CHECK_LAUNCH("ns_swiglu");
        return NS_OK;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == NS_F32)
        NS_LAUNCH((swiglu_kernel<float>), blocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter, block, total);
    else if (dtype == NS_BF16)
        NS_LAUNCH((swiglu_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block, total);
    else
        NS_FAIL(NS_ERR_ARGUMENT, "ns_swiglu: unknown dtype %d", dtype);
    NS_CHECK_LAUNCH("ns_swiglu");
    return NS_OK;
}
