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

// Activations are written by the preceding kernel: read through L2 (never a stale L1 line), after the wait.
__device__ __forceinline__ uint4 ldg_plain(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
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
                                   int epilogue, int prefetch, int ksplit, float* __restrict__ scratch,
                                   int* __restrict__ counters) {
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

    // grid.y splits K between blocks, the warps of a block split the block's share
    const int kblock = blockIdx.y * k_per_warp * n_warps;
    const int kbeg = min(K, kblock + warp * k_per_warp);
    const int kend = min(K, kbeg + k_per_warp);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // The weights are constant, so everything that touches only W happens before the wait on the
    // preceding kernel (whose output is A) and overlaps its tail: the first U steps are loaded into
    // registers and the rest of this warp's range is pulled into L2.
    uint4 wa[U][RT], wb[U][RT], xa[U][NT];

#define SKINNY_LOAD(KBASE)                                                 \
    _Pragma("unroll") for (int u = 0; u < U; ++u) {                        \
        const int kk = (KBASE) + u * 32 + t * 8;                           \
        const bool ok = kk < kend;                                         \
        _Pragma("unroll") for (int r = 0; r < RT; ++r) {                   \
            wa[u][r] = ok ? ldg_stream(wrow_a[r] + kk) : zero;             \
            wb[u][r] = ok ? ldg_stream(wrow_b[r] + kk) : zero;             \
        }                                                                  \
    }
    // activations of the same steps, issued right behind the weights so both are in flight together
#define SKINNY_LOAD_A(KBASE)                                                        \
    _Pragma("unroll") for (int u = 0; u < U; ++u) {                                 \
        const int kk = (KBASE) + u * 32 + t * 8;                                    \
        const bool ok = kk < kend;                                                  \
        _Pragma("unroll") for (int n = 0; n < NT; ++n)                              \
            xa[u][n] = (ok && arow_ok[n]) ? ldg_plain(arow[n] + kk) : zero;         \
    }

    SKINNY_LOAD(kbeg)
    {
        const int kpre = kbeg + 32 * U;                     // multiple of 32 elements = 64 bytes
        if (prefetch && kpre < kend) {
            const int lines = (kend - kpre + 63) / 64;      // 128-byte lines per row
            for (int idx = lane; idx < R * lines; idx += 32) {
                const int r = idx / lines, line = idx - r * lines;
                const int row = min(row0 + r, N - 1);
                const bf16* p = W + (size_t)row * ldw + kpre + line * 64;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
            }
        }
    }
    pdl_trigger();
    pdl_wait();
    for (int k0 = kbeg; k0 < kend; k0 += 32 * U) {
        if (k0 != kbeg) {
            SKINNY_LOAD(k0)
        }
        SKINNY_LOAD_A(k0)
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    mma_bf16_16816(acc[r][n], wa[u][r].x, wb[u][r].x, wa[u][r].y, wb[u][r].y, xa[u][n].x, xa[u][n].y);
                    mma_bf16_16816(acc[r][n], wa[u][r].z, wb[u][r].z, wa[u][r].w, wb[u][r].w, xa[u][n].z, xa[u][n].w);
                }
            }
        }
    }
#undef SKINNY_LOAD_A
#undef SKINNY_LOAD

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

    // With K split between blocks, each block leaves its [rows x M] partial in `scratch`; the last
    // block of a tile to arrive (a counter per tile, no waiting) adds the partials in split order,
    // so the sum does not depend on which block came last.
    const float* src = red;
    int n_src = n_warps;
    size_t src_stride = (size_t)R * RS;
    if (ksplit > 1) {
        __shared__ int s_last;
        float* mine_g = scratch + ((size_t)blockIdx.x * ksplit + blockIdx.y) * R * RS;
        for (int idx = threadIdx.x; idx < R * MP; idx += blockDim.x) {
            const int m = idx / R, r = idx - m * R;
            float v = 0.0f;
            for (int w = 0; w < n_warps; ++w) v += red[((size_t)w * R + r) * RS + m];
            mine_g[r * RS + m] = v;
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicAdd(&counters[blockIdx.x], 1) == ksplit - 1;
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        if (threadIdx.x == 0) counters[blockIdx.x] = 0;       // ready for the next launch
        src = scratch + (size_t)blockIdx.x * ksplit * R * RS;
        n_src = ksplit;
    }
    auto total = [&](int r, int m) {
        float v = 0.0f;
        if (ksplit > 1) {
            for (int w = 0; w < n_src; ++w) v += __ldcg(src + (size_t)w * src_stride + r * RS + m);
        } else {
            for (int w = 0; w < n_src; ++w) v += src[(size_t)w * src_stride + r * RS + m];
        }
        return v;
    };

    if (epilogue == EPI_SWIGLU) {
        constexpr int PAIRS = R / 2;
        for (int idx = threadIdx.x; idx < PAIRS * MP; idx += blockDim.x) {
            const int m = idx / PAIRS, p = idx - m * PAIRS;
            const int row = row0 + 2 * p;
            if (m >= M || row + 1 >= N) continue;
            store_from_f32(C, c_dtype, (size_t)m * ldc + (row >> 1), silu_mul_fast(total(2 * p, m), total(2 * p + 1, m)));
        }
    } else {
        for (int idx = threadIdx.x; idx < R * MP; idx += blockDim.x) {
            const int m = idx / R, r = idx - m * R;
            const int row = row0 + r;
            if (m >= M || row >= N) continue;
            const float v = total(r, m);
            const size_t o = (size_t)m * ldc + row;
            if (epilogue == EPI_ACCUMULATE)
                reinterpret_cast<float*>(C)[o] += v;
            else
                store_from_f32(C, c_dtype, o, v);
        }
    }
}

// Overrides of the plan for tests and experiments: 0 keeps the built-in choice.  An override holds
// for ONE call of a product entry point (the next one, which clears it when it returns, whether or
// not it launched), so nothing a test sets can outlive that test; bfi_skinny_gemm_scratch, which
// only asks for a plan's sizes, sees the pending override and leaves it standing.
static int g_tune_warps = 0;
static int g_tune_prefetch = 0;
static int g_tune_ksplit = 0;
extern "C" int bfi_skinny_tune_next(int warps, int prefetch, int ksplit) {
    g_tune_warps = warps;
    g_tune_prefetch = prefetch;
    g_tune_ksplit = ksplit;
    return 0;
}
struct SkinnyTuneScope {       // clears the override when the entry point that owns it returns
    bool owner;
    explicit SkinnyTuneScope(bool o) : owner(o) {}
    ~SkinnyTuneScope() {
        if (owner) g_tune_warps = g_tune_prefetch = g_tune_ksplit = 0;
    }
};
static int g_skinny_entry_depth = 0;

// The plan of a launch: warps per block, split of K between blocks, scratch it needs.
struct SkinnyPlan {
    int tiles, warps, ksplit, k_per_warp;
    size_t smem;
    long scratch_floats;
    int counters;
};

static SkinnyPlan plan_skinny(int rows_per_tile, int m_pad, int N, int K, bool allow_split) {
    SkinnyPlan p;
    p.tiles = (N + rows_per_tile - 1) / rows_per_tile;
    // many tiles: small blocks, several per SM; few tiles: wider blocks and K split between blocks
    const int sms = bfi_sm_count();
    p.warps = p.tiles >= 4 * sms ? 4 : 8;
    if (g_tune_warps > 0) p.warps = g_tune_warps;
    while (p.warps > 1 && K / p.warps < 64) p.warps >>= 1;
    p.ksplit = 1;
    if (allow_split && p.tiles < 2 * sms) {
        p.ksplit = (2 * sms + p.tiles - 1) / p.tiles;   // about two blocks per SM
        while (p.ksplit > 1 && K / (p.ksplit * p.warps) < 128) --p.ksplit;
    }
    if (g_tune_ksplit > 0 && allow_split) p.ksplit = g_tune_ksplit;
    int per = (K + p.ksplit * p.warps - 1) / (p.ksplit * p.warps);
    p.k_per_warp = ((per + 31) / 32) * 32;
    p.smem = (size_t)p.warps * rows_per_tile * (m_pad + 1) * sizeof(float);
    p.scratch_floats = p.ksplit > 1 ? (long)p.tiles * p.ksplit * rows_per_tile * (m_pad + 1) : 0;
    p.counters = p.ksplit > 1 ? p.tiles : 0;
    return p;
}

template <int NT, int RT, int U>
static int launch_skinny(const bf16* A, long lda, const bf16* W, long ldw, void* C, int c_dtype, long ldc, int M, int N,
                         int K, int epilogue, float* scratch, long scratch_floats, int* counters, int n_counters,
                         cudaStream_t stream) {
    constexpr int R = RT * 16;
    SkinnyPlan p = plan_skinny(R, NT * 8, N, K, scratch != nullptr && counters != nullptr);
    if (p.ksplit > 1 && (p.scratch_floats > scratch_floats || p.counters > n_counters))
        return bfi_fail("skinny_gemm: scratch too small: need %ld floats and %d counters, got %ld and %d",
                        p.scratch_floats, p.counters, scratch_floats, n_counters);
    auto kernel = skinny_gemm_kernel<NT, RT, U>;
    if (p.smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) return bfi_fail("skinny_gemm: cannot reserve %zu bytes of shared memory: %s", p.smem,
                                              cudaGetErrorString(e));
    }
    bfi_launch(kernel, dim3(p.tiles, p.ksplit), dim3(p.warps * 32), p.smem, stream, A, lda, W, ldw, C, c_dtype, ldc, M, N,
               K, p.k_per_warp, epilogue, g_tune_prefetch, p.ksplit, scratch, counters);
    return bfi_check_launch("skinny_gemm");
}

static inline bool skinny_wide(int M, int N) { return N >= 9600 && M <= 32; }
static inline int skinny_nt(int M) { return M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8)); }

// Scratch a call may use: sizes[0] floats, sizes[1] int counters (which must start at zero and are
// left at zero by every call).  Zero means the shape never splits K.
extern "C" int bfi_skinny_gemm_scratch(int M, int N, int K, long* sizes) {
    const int rows = skinny_wide(M, N) ? 32 : 16;
    SkinnyPlan p = plan_skinny(rows, skinny_nt(M) * 8, N, K, true);
    sizes[0] = p.scratch_floats;
    sizes[1] = p.counters;
    return 0;
}

// The checks every entry point makes before it puts anything on the stream: 0 when the call may
// go ahead (or has nothing to do, M == 0), 1 on an error (the text is left for bfi_last_error), 2
// when the shape is not one the kernel takes.
static int skinny_check_args(const void* A, long lda, const void* W, long ldw, int c_dtype, int M, int N, int K,
                             int epilogue) {
    BFI_REQUIRE(dtype_ok(c_dtype), "skinny_gemm: unknown output dtype code %d", c_dtype);
    BFI_REQUIRE(M >= 0 && N > 0 && K > 0, "skinny_gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    BFI_REQUIRE(epilogue >= 0 && epilogue <= 2, "skinny_gemm: unknown epilogue %d", epilogue);
    if (epilogue == EPI_ACCUMULATE) BFI_REQUIRE(c_dtype == BFI_F32, "skinny_gemm: accumulation needs a float32 output");
    if (epilogue == EPI_SWIGLU) BFI_REQUIRE(N % 2 == 0, "skinny_gemm: the gated epilogue needs an even N, got %d", N);
    if (M == 0) return 0;
    // 16-byte loads: K a multiple of 8, rows and bases 16-byte aligned
    if (M > 64 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 2;
    return 0;
}

// Returns 0 on success, 1 on error, and 2 when the shape is not taken (nothing launched; the
// caller uses the general kernel).
extern "C" int bfi_skinny_gemm_bf16(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype, long ldc,
                                    int M, int N, int K, int epilogue, float* scratch, long scratch_floats,
                                    int* counters, int n_counters, cudaStream_t stream) {
    SkinnyTuneScope scope(g_skinny_entry_depth == 0);
    const int verdict = skinny_check_args(A, lda, W, ldw, c_dtype, M, N, K, epilogue);
    if (verdict != 0 || M == 0) return verdict;
    const bf16* a = (const bf16*)A;
    const bf16* w = (const bf16*)W;
    const bool wide = skinny_wide(M, N);   // many rows: two m-tiles per block halve the activation traffic
#define BFI_SKINNY(NT, U1, U2)                                                                                     \
    return wide ? launch_skinny<NT, 2, U2>(a, lda, w, ldw, C, c_dtype, ldc, M, N, K, epilogue, scratch,            \
                                           scratch_floats, counters, n_counters, stream)                           \
                : launch_skinny<NT, 1, U1>(a, lda, w, ldw, C, c_dtype, ldc, M, N, K, epilogue, scratch,            \
                                           scratch_floats, counters, n_counters, stream);
    if (M <= 8) { BFI_SKINNY(1, 4, 4) }
    if (M <= 16) { BFI_SKINNY(2, 4, 4) }
    if (M <= 32) { BFI_SKINNY(4, 2, 2) }
    return launch_skinny<8, 1, 2>(a, lda, w, ldw, C, c_dtype, ldc, M, N, K, epilogue, scratch, scratch_floats, counters,
                                  n_counters, stream);
#undef BFI_SKINNY
}

// ------------------------------------------------------------------------------------------
// The same product for callers that cannot allocate: scratch in the library's own device image.
// See no_alloc.h for the contract.
// ------------------------------------------------------------------------------------------
#include "no_alloc.h"

static __device__ __align__(256) float bfi_static_scratch[BFI_STATIC_SCRATCH_FLOATS];

#define BFI_MAX_DEVICES 64
static float* g_static_scratch_addr[BFI_MAX_DEVICES] = {nullptr};

// The array's name is only a host-side handle; kernels need its address on the current device.
static int static_scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return bfi_fail("skinny_gemm_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= BFI_MAX_DEVICES) return bfi_fail("skinny_gemm_static: device index %d out of range", dev);
    if (g_static_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, bfi_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return bfi_fail("skinny_gemm_static: cannot find the scratch array on device %d: %s", dev,
                            cudaGetErrorString(e));
        g_static_scratch_addr[dev] = static_cast<float*>(p);
    }
    *out = g_static_scratch_addr[dev];
    return 0;
}

extern "C" int bfi_skinny_gemm_bf16_static(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype,
                                           long ldc, int M, int N, int K, int epilogue, cudaStream_t stream) {
    SkinnyTuneScope scope(true);
    struct Depth {
        Depth() { ++g_skinny_entry_depth; }
        ~Depth() { --g_skinny_entry_depth; }
    } depth;                                   // the inner call must not clear the override before it planned
    // every refusal comes before the first thing this call puts on the stream
    const int verdict = skinny_check_args(A, lda, W, ldw, c_dtype, M, N, K, epilogue);
    if (verdict != 0 || M == 0) return verdict;
    long need[2] = {0, 0};
    bfi_skinny_gemm_scratch(M, N, K, need);
    const long room = (long)BFI_STATIC_SCRATCH_FLOATS - BFI_STATIC_COUNTER_SLOTS;
    BFI_REQUIRE(need[0] <= room && need[1] <= BFI_STATIC_COUNTER_SLOTS,
                "skinny_gemm_static: M=%d N=%d K=%d needs %ld floats of scratch and %ld counters; the built-in array "
                "holds %ld and %d",
                M, N, K, need[0], need[1], room, BFI_STATIC_COUNTER_SLOTS);
    float* base = nullptr;
    int rc = static_scratch_address(&base);
    if (rc) return rc;
    int* counters = reinterpret_cast<int*>(base);
    float* partials = base + BFI_STATIC_COUNTER_SLOTS;
    if (need[1] > 0) {
        // whatever an earlier call left behind, the counters of this call start at zero
        cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)need[1] * sizeof(int), stream);
        if (e != cudaSuccess) return bfi_fail("skinny_gemm_static: clearing the counters failed: %s", cudaGetErrorString(e));
    }
    return bfi_skinny_gemm_bf16(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, partials, room, counters,
                                BFI_STATIC_COUNTER_SLOTS, stream);
}
