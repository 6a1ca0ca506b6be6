// Shared helpers of the sm_100a kernel library: storage types, conversions, reductions and the
// error convention of the exported C functions.
//
// Every exported function returns 0 on success.  On failure it returns a non-zero code and
// leaves a message that bfi_last_error() hands out; nothing is launched in that case.
// Storage types are named by code: 0 = float32, 1 = bfloat16.  Arithmetic is float32 everywhere.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#define BFI_F32 0
#define BFI_BF16 1

#define BFI_PAGE_TOKENS 64

// status word bits (device side checks record and skip; they never trap)
#define BFI_STATUS_BAD_TOKEN 1
#define BFI_STATUS_NO_PAGE 2
#define BFI_STATUS_BAD_POSITION 4

typedef __nv_bfloat16 bf16;

extern "C" const char* bfi_last_error();
int bfi_fail(const char* fmt, ...);
int bfi_check_launch(const char* what);
int bfi_sm_count();

// Programmatic dependent launch.  When enabled, every kernel is launched with the attribute that
// lets it start while its predecessor in the stream drains.  A kernel may touch nothing but
// constant weights before pdl_wait(), which returns once the predecessor has completed and its
// writes are visible; without the attribute the instruction returns at once.
extern int g_bfi_pdl;

#ifdef BFI_TRACE
// Timeline of a step, for builds made with -DBFI_TRACE (environment variable BFI_B200_TRACE=1): the
// first thread of every block stamps the global timer when the block starts (0), when its wait for
// the kernel before it returns (1) and, in the kernels that say so, when it is done (2).  Records
// are {grid id << 32 | what << 28 | linear block id, nanoseconds}; every source file has a buffer of
// its own (BFI_TRACE_EXPORT at its end gives it a reader).
#define BFI_TRACE_RECORDS (1 << 18)
static __device__ unsigned long long g_bfi_trace[2 + 2 * BFI_TRACE_RECORDS];
__device__ __forceinline__ void bfi_trace(unsigned what) {
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        unsigned long long now, gid;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        asm volatile("mov.u64 %0, %%gridid;" : "=l"(gid));
        const unsigned long long i = atomicAdd(&g_bfi_trace[0], 1ull);
        if (i < BFI_TRACE_RECORDS) {
            const unsigned long long blk = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
            g_bfi_trace[2 + 2 * i] = (gid << 32) | ((unsigned long long)what << 28) | (blk & 0xFFFFFFFull);
            g_bfi_trace[3 + 2 * i] = now;
        }
    }
}
#define BFI_TRACE_END() bfi_trace(2)
#define BFI_TRACE_EXPORT(name)                                                                                   \
    extern "C" long bfi_trace_read_##name(unsigned long long* host, long cap) {                                  \
        unsigned long long head[2] = {0, 0};                                                                     \
        cudaDeviceSynchronize();                                                                                 \
        cudaMemcpyFromSymbol(head, g_bfi_trace, sizeof(head));                                                   \
        long n = (long)(head[0] < BFI_TRACE_RECORDS ? head[0] : BFI_TRACE_RECORDS);                              \
        if (n > cap) n = cap;                                                                                    \
        if (n > 0) cudaMemcpyFromSymbol(host, g_bfi_trace, (size_t)n * 16, 16);                                  \
        head[0] = 0;                                                                                             \
        cudaMemcpyToSymbol(g_bfi_trace, head, sizeof(head));                                                     \
        return n;                                                                                                \
    }
#else
#define BFI_TRACE_END()
#define BFI_TRACE_EXPORT(name)
#endif

__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
#ifdef BFI_TRACE
    bfi_trace(1);
#endif
}
__device__ __forceinline__ void pdl_trigger() {
#ifdef BFI_TRACE
    bfi_trace(0);
#endif
    asm volatile("griddepcontrol.launch_dependents;");
}

template <typename... KArgs, typename... Args>
static inline cudaError_t bfi_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_bfi_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define BFI_REQUIRE(cond, ...)                  \
    do {                                        \
        if (!(cond)) return bfi_fail(__VA_ARGS__); \
    } while (0)

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Loads a value of storage type `dtype` (runtime code) at element index i.
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
    return dtype == BFI_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
    if (dtype == BFI_F32)
        reinterpret_cast<float*>(p)[i] = v;
    else
        reinterpret_cast<bf16*>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

static inline int dtype_size(int dtype) { return dtype == BFI_F32 ? 4 : 2; }
static inline bool dtype_ok(int dtype) { return dtype == BFI_F32 || dtype == BFI_BF16; }
