// Shared helpers of the sm_100a kernels: element types, error reporting, warp and block
// reductions.  Every exported function returns 0 on success and a non-zero code otherwise;
// ns_last_error() gives the text of the last failure on the calling thread.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define NS_API extern "C" __attribute__((visibility("default")))

enum NsDtype { NS_F32 = 0, NS_BF16 = 1 };

enum NsStatus {
    NS_OK = 0,
    NS_ERR_UNSUPPORTED = 1,  // a size or option that this kernel refuses
    NS_ERR_CUDA = 2,         // a CUDA call failed
    NS_ERR_ARGUMENT = 3,     // inconsistent arguments
};

// set by ns_fail(), read through ns_last_error()
extern thread_local char ns_error_text[512];

#define NS_FAIL(code, ...)                                        \
    do {                                                          \
        snprintf(ns_error_text, sizeof(ns_error_text), __VA_ARGS__); \
        return (code);                                            \
    } while (0)

#define NS_CHECK_LAUNCH(name)                                                             \
    do {                                                                                  \
        cudaError_t e_ = cudaGetLastError();                                              \
        if (e_ != cudaSuccess) NS_FAIL(NS_ERR_CUDA, "%s: %s", name, cudaGetErrorString(e_)); \
    } while (0)

#define NS_CUDA(call)                                                                       \
    do {                                                                                    \
        cudaError_t e_ = (call);                                                            \
        if (e_ != cudaSuccess) NS_FAIL(NS_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

// ---- element access: everything is computed in float -----------------------------------
__device__ __forceinline__ float ns_ld(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ns_ld(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void ns_st(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void ns_st(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// eight consecutive elements with 16-byte accesses (the address must be 16-byte aligned)
__device__ __forceinline__ void ld8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void st8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ float ns_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float ns_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum in a fixed order (warp tree, then warp 0 over the warp partials), so the
// result does not depend on anything but the block size.  `scratch` holds 32 floats.
__device__ __forceinline__ float ns_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = ns_warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nwarp) ? scratch[threadIdx.x] : 0.f;
    if (warp == 0) {
        t = ns_warp_sum(t);
        if (lane == 0) scratch[0] = t;
    }
    __syncthreads();
    return scratch[0];
}
__device__ __forceinline__ float ns_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = ns_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < nwarp) ? scratch[threadIdx.x] : -INFINITY;
    if (warp == 0) {
        t = ns_warp_max(t);
        if (lane == 0) scratch[0] = t;
    }
    __syncthreads();
    return scratch[0];
}

// ---- launches ------------------------------------------------------------------------------
// Every kernel of this library is launched with programmatic stream serialisation allowed: a
// kernel may be scheduled while its predecessor in the stream is still running, and it calls
// ns_pdl_wait() before it touches anything the predecessor wrote (or writes anything the
// predecessor may read).  What runs before that wait - barrier set-up, TMEM allocation, the first
// weight tiles of a matrix product - overlaps the predecessor.  ns_set_pdl(0) turns this off.
// Every block waits before it returns, also one that has nothing to do (a padding row): a grid none of
// whose blocks waited would complete while its predecessor still runs, and the wait of ITS successor,
// which covers the grid directly before it only, would no longer mean "everything earlier is done".
extern int ns_pdl_enabled;

__device__ __forceinline__ void ns_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ns_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t ns_launch_impl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ns_pdl_enabled ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#define NS_LAUNCH(kernel, grid, block, smem, stream, ...) \
    (void)ns_launch_impl(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__)
