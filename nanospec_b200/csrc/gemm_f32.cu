// True 32-bit matrix product on the CUDA cores: y[M, N] = x[M, K] * w[N, K]^T.
//
// No tensor cores and no reduced-precision mode: every product and sum is an fp32 FMA.
// Each output element is accumulated by one thread over k = 0..K-1 in ascending order, so
// its value does not depend on M, on the tile it falls in, or on what else is in the batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <bool kAligned>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int M, int N, int K,
                int ldx, int ldw, int ldy) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = tid & 15, ty = tid >> 4;  // thread's 4x4 patch: rows ty*4.., cols tx*4..

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // loading: 64 rows x 16 k per operand = 1024 floats = 256 threads x 4 consecutive k
    const int lrow = tid >> 2, lk = (tid & 3) * 4;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            const int gm = m0 + lrow;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (gm < M) {
                const float* p = x + (size_t)gm * ldx + k0 + lk;
                if (kAligned && k0 + lk + 3 < K) {
                    const float4 t = *reinterpret_cast<const float4*>(p);
                    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (k0 + lk + i < K) v[i] = p[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) xs[lk + i][lrow] = v[i];
        }
        {
            const int gn = n0 + lrow;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (gn < N) {
                const float* p = w + (size_t)gn * ldw + k0 + lk;
                if (kAligned && k0 + lk + 3 < K) {
                    const float4 t = *reinterpret_cast<const float4*>(p);
                    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (k0 + lk + i < K) v[i] = p[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) ws[lk + i][lrow] = v[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) y[(size_t)gm * ldy + gn] = acc[i][j];
        }
    }
}

}  // namespace

// x: [M, K] with row stride ldx; w: [N, K] with row stride ldw; y: [M, N] with row stride ldy.
NS_API int ns_gemm_f32(const float* x, const float* w, float* y, int M, int N, int K, int ldx, int ldw, int ldy,
                       cudaStream_t stream) {
    if (M <= 0 || N <= 0) return NS_OK;
    if (K <= 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_gemm_f32: K=%d", K);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_f32: M=%d exceeds 65535 row tiles", M);
    const bool aligned = (ldx % 4 == 0) && (ldw % 4 == 0) && (((uintptr_t)x | (uintptr_t)w) % 16 == 0);
    if (aligned)
        NS_LAUNCH((gemm_f32_kernel<true>), grid, 256, 0, stream, x, w, y, M, N, K, ldx, ldw, ldy);
    else
        NS_LAUNCH((gemm_f32_kernel<false>), grid, 256, 0, stream, x, w, y, M, N, K, ldx, ldw, ldy);
    NS_CHECK_LAUNCH("ns_gemm_f32");
    return NS_OK;
}
