// Warp-level matrix helpers shared by the attention kernels: cp.async copies into shared
// memory, ldmatrix fragment loads, the bf16 m16n8k16 tensor-core instruction, and the padded
// tile layout that keeps ldmatrix free of bank conflicts.
#pragma once

#include "common.cuh"

__device__ __forceinline__ uint32_t ns_smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// 16-byte asynchronous copy global -> shared; copies `valid ? 16 : 0` bytes and zero-fills the rest
__device__ __forceinline__ void ns_cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
    const uint32_t d = ns_smem_u32(smem_dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gmem_src), "r"(n) : "memory");
}
__device__ __forceinline__ void ns_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void ns_cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ns_ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(ns_smem_u32(smem_row)));
}
__device__ __forceinline__ void ns_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(ns_smem_u32(smem_row)));
}

// d (16x8, fp32) += a (16x16, bf16, row) * b (16x8, bf16, col)
__device__ __forceinline__ void ns_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x for x <= 0 in one instruction (ex2.approx, about 2 ulp): the softmax weights of the tensor-core kernels
__device__ __forceinline__ float ns_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t ns_pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Tiles in shared memory are rows of D bf16 padded by 8 elements (16 bytes): for D a multiple
// of 16 the row stride is an odd number of 16-byte units, so the 8 rows that one ldmatrix phase
// reads fall in 8 different 16-byte bank groups.
template <int D>
struct NsTile {
    static constexpr int kStride = D + 8;
    __device__ static __forceinline__ __nv_bfloat16* at(__nv_bfloat16* tile, int row, int col) {
        return tile + row * kStride + col;
    }
};
