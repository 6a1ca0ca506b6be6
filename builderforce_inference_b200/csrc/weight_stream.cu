// A measuring stick for the few-row products: the kernel reads a bfloat16 weight matrix W[N, K]
// once, the way those products do -- tiles of 128 rows x 64 columns by TMA (128-byte swizzle) into
// a ring in shared memory, an mbarrier per stage -- and does nothing with it: one thread waits for
// each tile and hands its stage back.  What a launch of it takes is what a product of that shape
// cannot beat with the same ring, whatever its tensor-core work and epilogue cost
// (`python bench.py --kernel weight_stream --shape gateup`).  Every wait is bounded.
#include "tcgen05.cuh"

#define WS_STAGE_BYTES (128 * 64 * 2)
#define WS_MAX_STAGES 12

__global__ void __launch_bounds__(64) weight_stream_kernel(const __grid_constant__ CUtensorMap map_w, int kblocks_per_split,
                                                          int total_kblocks, int stages, int* __restrict__ status,
                                                          unsigned long long* __restrict__ sink) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)stages * WS_STAGE_BYTES);
    uint64_t* empty = full + WS_MAX_STAGES;
    const uint32_t spin_limit = TC_SPIN_LIMIT;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();
    const int kb_beg = blockIdx.y * kblocks_per_split;
    const int n_kb = max(0, min(total_kblocks, kb_beg + kblocks_per_split) - kb_beg);
    if (threadIdx.x == 0) {
        for (int i = 0; i < n_kb; ++i) {
            const int s = i % stages;
            if (i >= stages && !MBAR_WAIT(&empty[s], (uint32_t)(((i / stages) & 1) ^ 1))) {
                atomicOr(status, BFI_STATUS_TIMEOUT);
                break;
            }
            mbar_expect_tx(&full[s], WS_STAGE_BYTES);
            tma_load_2d(smem + (size_t)s * WS_STAGE_BYTES, &map_w, (kb_beg + i) * 64, blockIdx.x * 128, &full[s]);
        }
    } else if (threadIdx.x == 32) {
        unsigned long long seen = 0;
        for (int i = 0; i < n_kb; ++i) {
            const int s = i % stages;
            if (!MBAR_WAIT(&full[s], (uint32_t)((i / stages) & 1))) {
                atomicOr(status, BFI_STATUS_TIMEOUT);
                break;
            }
            seen += *reinterpret_cast<const unsigned long long*>(smem + (size_t)s * WS_STAGE_BYTES);
            mbar_arrive(&empty[s]);
        }
        if (seen == 0x0123456789abcdefull) *sink = seen;         // keeps the reads alive
    }
    pdl_wait();
    __syncthreads();
}

// Streams W[n, k] (row stride ldw elements) once: n/128 row tiles x `ksplit` ranges of k, each
// block with a ring of `stages` 16 KB tiles.  Returns 0 on success, 1 on error, 2 when TMA cannot
// address the operand.  `status` gets BFI_STATUS_TIMEOUT if a wait ran out; `sink` points at 8 bytes.
extern "C" int bfi_weight_stream_bf16(const void* W, long ldw, int n, int k, int stages, int ksplit, int* status,
                                      unsigned long long* sink, cudaStream_t stream) {
    BFI_REQUIRE(n > 0 && k > 0 && status != nullptr && sink != nullptr, "weight_stream: bad sizes or no status word");
    BFI_REQUIRE(stages >= 1 && stages <= WS_MAX_STAGES && ksplit >= 1, "weight_stream: 1..%d stages, at least one split",
                WS_MAX_STAGES);
    if (k % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)W & 15)) return 2;
    CUtensorMap mw;
    int rc = bfi_tensor_map_bf16(W, n, k, ldw, 128, &mw);
    if (rc) return rc;
    const int total_kblocks = (k + 63) / 64;
    const int per_split = (total_kblocks + ksplit - 1) / ksplit;
    const size_t smem = (size_t)stages * WS_STAGE_BYTES + 1024 + 2 * WS_MAX_STAGES * sizeof(uint64_t);
    static bool configured = false;
    if (!configured) {
        const size_t most = (size_t)WS_MAX_STAGES * WS_STAGE_BYTES + 1024 + 2 * WS_MAX_STAGES * sizeof(uint64_t);
        cudaError_t e = cudaFuncSetAttribute(weight_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
        if (e != cudaSuccess)
            return bfi_fail("weight_stream: cannot reserve %zu bytes of shared memory: %s", most, cudaGetErrorString(e));
        configured = true;
    }
    bfi_launch(weight_stream_kernel, dim3((n + 127) / 128, (total_kblocks + per_split - 1) / per_split), dim3(64), smem, stream,
               mw, per_split, total_kblocks, stages, status, sink);
    return bfi_check_launch("weight_stream");
}
