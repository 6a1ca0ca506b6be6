// Decode-time matrix product for few rows of activations (M <= 64), bfloat16 x bfloat16 with
// float32 accumulation: C[M,N] = A[M,K] * W[N,K]^T.  The step is bound by reading W once from
// HBM, so the kernel is a weight streamer: every lane issues 16-byte loads straight from global
// memory into the registers that feed the tensor cores, many of them in flight, and W never
// passes through shared memory.
//
// Roles are swapped with respect to the usual GEMM: 16 rows of W are the "M" side of
// mma.sync.m16n8k16 and 8 rows of activations are its "N" side, so a batch of up to 64 rows costs
// 8 n-tiles per weight fragment.  The k index is permuted inside each group of 32 (a lane owns 8
// consecutive k of its row, used as k-slots {2t,2t+1,2t+8,2t+9} of two MMAs); A and W use the same
// permutation, so the dot products are unchanged while every load is 16 bytes and 4 lanes cover
// 64 contiguous bytes of a row.
//
// A block owns RT*16 rows of W; its warps split K into contiguous ranges and their partial sums
// are added in a fixed order through shared memory, so the result does not depend on timing.
//
// Epilogues as in gemm_simt.cu: 0 store, 1 add into the float32 residual, 2 SiLU(gate)*up over
// interleaved rows.
#include "common.cuh"

#define EPI_STORE 0
#define EPI_ACCUMULATE 1
#define EPI_SWIGLU 2

__device__ __forceinline__ float silu_mul_fast(float g, float u) {
    float s;
    if (g >= 0.0f) {
        s = 1.0f / (1.0f + __expf(-g));
    } else {
        const float z = __expf(g);
        s = z / (1.0f + z);
    }
    return g * s * u;
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 ldg_cached(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: n-tiles of 8 activation rows (M <= 8*NT).  RT: m-tiles of 16 W rows per block.
// U: steps of 32 k whose weight loads are issued together.
template <int NT, int RT, int U>
__global__ void skinny_gemm_kernel(const bf16* __restrict__ A, long lda, const bf16* __restrict__ W, long ldw,
                                   void* __restrict__ C, int c_dtype, long ldc, int M, int N, int K, int k_per_warp,
                                   int epilogue) {
    extern __shared__ float red[];   // [warps][RT*16][NT*8 + 1]
    constexpr int R = RT * 16;
    constexpr int MP = NT * 8;
    constexpr int RS = MP + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_warps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * R;

    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[r][n][i] = 0.0f;

    const bf16* wrow_a[RT];
    const bf16* wrow_b[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const int ra = min(row0 + r * 16 + g, N - 1);       // rows past N are loaded but never stored
        const int rb = min(row0 + r * 16 + g + 8, N - 1);
        wrow_a[r] = W + (size_t)ra * ldw;
        wrow_b[r] = W + (size_t)rb * ldw;
    }
    const bf16* arow[NT];
    bool arow_ok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const int m = n * 8 + g;
        arow_ok[n] = m < M;
        arow[n] = A + (size_t)(arow_ok[n] ? m : 0) * lda;
    }

    const int kbeg = warp * k_per_warp;
    const int kend = min(K, kbeg + k_per_warp);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    for (int k0 = kbeg; k0 < kend; k0 += 32 * U) {
        uint4 wa[U][RT], wb[U][RT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kk = k0 + u * 32 + t * 8;
            const bool ok = kk < kend;
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                wa[u][r] = ok ? ldg_stream(wrow_a[r] + kk) : zero;
                wb[u][r] = ok ? ldg_stream(wrow_b[r] + kk) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kk = k0 + u * 32 + t * 8;
            const bool ok = kk < kend;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const uint4 x = (ok && arow_ok[n]) ? ldg_cached(arow[n] + kk) : zero;
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    mma_bf16_16816(acc[r][n], wa[u][r].x, wb[u][r].x, wa[u][r].y, wb[u][r].y, x.x, x.y);
                    mma_bf16_16816(acc[r][n], wa[u][r].z, wb[u][r].z, wa[u][r].w, wb[u][r].w, x.z, x.w);
                }
            }
        }
    }

    // partial sums of this warp -> shared memory.  c0:(row g, col 2t) c1:(g, 2t+1) c2:(g+8, 2t) c3:(g+8, 2t+1)
    float* mine = red + (size_t)warp * R * RS;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int col = n * 8 + 2 * t;
            mine[(r * 16 + g) * RS + col] = acc[r][n][0];
            mine[(r * 16 + g) * RS + col + 1] = acc[r][n][1];
            mine[(r * 16 + g + 8) * RS + col] = acc[r][n][2];
            mine[(r * 16 + g + 8) * RS + col + 1] = acc[r][n][3];
        }
    __syncthreads();

    if (epilogue == EPI_SWIGLU) {
        constexpr int PAIRS = R / 2;
        for (int idx = threadIdx.x; idx < PAIRS * MP; idx += blockDim.x) {
            const int m = idx / PAIRS, p = idx - m * PAIRS;
            const int row = row0 + 2 * p;
            if (m >= M || row + 1 >= N) continue;
            float gate = 0.0f, up = 0.0f;
            for (int w = 0; w < n_warps; ++w) {
                gate += red[((size_t)w * R + 2 * p) * RS + m];
                up += red[((size_t)w * R + 2 * p + 1) * RS + m];
            }
            store_from_f32(C, c_dtype, (size_t)m * ldc + (row >> 1), silu_mul_fast(gate, up));
        }
    } else {
        for (int idx = threadIdx.x; idx < R * MP; idx += blockDim.x) {
            const int m = idx / R, r = idx - m * R;
            const int row = row0 + r;
            if (m >= M || row >= N) continue;
            float v = 0.0f;
            for (int w = 0; w < n_warps; ++w) v += red[((size_t)w * R + r) * RS + m];
            const size_t o = (size_t)m * ldc + row;
            if (epilogue == EPI_ACCUMULATE)
                reinterpret_cast<float*>(C)[o] += v;
            else
                store_from_f32(C, c_dtype, o, v);
        }
    }
}

template <int NT, int RT, int U>
static int launch_skinny(const bf16* A, long lda, const bf16* W, long ldw, void* C, int c_dtype, long ldc, int M, int N,
                         int K, int epilogue, cudaStream_t stream) {
    constexpr int R = RT * 16;
    const int tiles = (N + R - 1) / R;
    // enough warps to keep ~16 per SM busy, each with at least 4 steps of 32 k
    int warps = 8;
    if ((long)tiles * 8 < 148L * 12 && K >= 16 * 128) warps = 16;
    while (warps > 1 && K / warps < 64) warps >>= 1;
    int k_per_warp = (K + warps - 1) / warps;
    k_per_warp = ((k_per_warp + 31) / 32) * 32;
    const size_t smem = (size_t)warps * R * (NT * 8 + 1) * sizeof(float);
    auto kernel = skinny_gemm_kernel<NT, RT, U>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return bfi_fail("skinny_gemm: cannot reserve %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
    }
    kernel<<<tiles, warps * 32, smem, stream>>>(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, k_per_warp, epilogue);
    return bfi_check_launch("skinny_gemm");
}

// Returns 0 on success, 1 on error, and 2 when the shape is not taken (nothing launched; the
// caller uses the general kernel).
extern "C" int bfi_skinny_gemm_bf16(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype, long ldc,
                                    int M, int N, int K, int epilogue, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(c_dtype), "skinny_gemm: unknown output dtype code %d", c_dtype);
    BFI_REQUIRE(M >= 0 && N > 0 && K > 0, "skinny_gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    BFI_REQUIRE(epilogue >= 0 && epilogue <= 2, "skinny_gemm: unknown epilogue %d", epilogue);
    if (epilogue == EPI_ACCUMULATE) BFI_REQUIRE(c_dtype == BFI_F32, "skinny_gemm: accumulation needs a float32 output");
    if (epilogue == EPI_SWIGLU) BFI_REQUIRE(N % 2 == 0, "skinny_gemm: the gated epilogue needs an even N, got %d", N);
    if (M == 0) return 0;
    // 16-byte loads: K a multiple of 8, rows and bases 16-byte aligned
    if (M > 64 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 2;
    const bf16* a = (const bf16*)A;
    const bf16* w = (const bf16*)W;
    const bool wide = N >= 9600;   // many rows: two m-tiles per block halve the activation traffic
#define BFI_SKINNY(NT, U)                                                                                          \
    return wide ? launch_skinny<NT, 2, U>(a, lda, w, ldw, C, c_dtype, ldc, M, N, K, epilogue, stream)              \
                : launch_skinny<NT, 1, U>(a, lda, w, ldw, C, c_dtype, ldc, M, N, K, epilogue, stream);
    if (M <= 8) { BFI_SKINNY(1, 4) }
    if (M <= 16) { BFI_SKINNY(2, 4) }
    if (M <= 32) { BFI_SKINNY(4, 2) }
    BFI_SKINNY(8, 2)
#undef BFI_SKINNY
}
