// Building blocks shared by the bfloat16 attention kernels: cp.async tiles of 64 cache rows in
// shared memory with an XOR swizzle, ldmatrix fragments, mma.sync.m16n8k16, ex2.approx.
#pragma once

#include "common.cuh"

#define AD_WARPS 4
#define AD_THREADS (AD_WARPS * 32)
#define AD_TILE 64          // keys per tile = tokens per page

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A tile in shared memory: [64 rows][D] bfloat16; the 16-byte chunk c of row r sits at chunk
// c ^ (r & 7), which makes the 8 row addresses of every ldmatrix fall into distinct banks.
template <int D>
__device__ __forceinline__ const bf16* tile_chunk(const bf16* tile, int row, int chunk) {
    return tile + row * D + ((chunk ^ (row & 7)) << 3);
}

template <int D>
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* src) {
    constexpr int CHUNKS = D / 8;                 // per row
    for (int i = threadIdx.x; i < AD_TILE * CHUNKS; i += AD_THREADS) {
        const int row = i / CHUNKS, c = i - row * CHUNKS;
        cp_async16(dst + row * D + ((c ^ (row & 7)) << 3), src + row * D + c * 8);
    }
}

