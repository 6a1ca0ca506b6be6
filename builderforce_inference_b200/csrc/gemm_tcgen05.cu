// bfloat16 matrix product on the fifth-generation tensor cores: C[M,N] = A[M,K] * W[N,K]^T with
// float32 accumulation in tensor memory.
//
// The roles are swapped with respect to the textbook GEMM: 128 rows of W are the M side of
// tcgen05.mma (one TMEM lane per output feature) and BT tokens are its N side (one TMEM column
// per token), so the same kernel serves prompts (BT = 256 tokens per tile) and decode batches
// (BT = 16..64), where the work is streaming W once: a ring of up to ten 16 KB weight tiles per
// SM is kept in flight by TMA.
//
//   warp 0     one lane issues the TMA loads of W and A tiles (128-byte swizzle) into the ring
//   warp 1     allocates tensor memory; one lane issues tcgen05.mma (4 per 64-wide k block) and
//              commits each block to the ring's "empty" barrier, the last one to "tmem_full"
//   warps 2-5  epilogue (2-9 in the many-row kernel, two per quarter of the lanes): tcgen05.ld of
//              their 32 lanes, then store / add into the float32 residual /
//              SiLU(gate)*up over interleaved rows.  With K split, the blocks of one tile form a
//              thread-block cluster: each leaves its partial tile in its own shared memory and
//              then adds, in split order, a share of the tile's tokens out of all the blocks'
//              shared memory (distributed shared memory), so nothing goes through global scratch
//              and the sum does not depend on timing
//
// Every wait on an mbarrier is bounded: a wait that runs out records BFI_STATUS_TIMEOUT in the
// status word, and the block drains its copies, frees its tensor memory and returns.
#include <mutex>
#include <unordered_map>

#include "tcgen05.cuh"

#define EPI_STORE 0
#define EPI_ACCUMULATE 1
#define EPI_SWIGLU 2

#define TC_ROWS 128           // W rows per tile (UMMA M)
#define TC_BK 64              // k elements per stage: one 128-byte swizzle row
#define TC_THREADS 192

// SiLU(g) * u for the bfloat16 path: g / (1 + e^-g) with the fast exponential and division
// (e^-g overflowing to infinity for very negative g gives -0, as it should).
__device__ __forceinline__ float silu_mul_tc(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

template <int BT>
struct TcConfig {
    static constexpr int STAGE_BYTES = TC_ROWS * TC_BK * 2 + BT * TC_BK * 2;
    // few tokens per tile (decode): two blocks share an SM, each with a ring of ~110 KB, so that a
    // grid a little larger than the SM count still runs in one wave; many tokens: one block per SM
    static constexpr int BUDGET = BT <= 64 ? 110 * 1024 : 196 * 1024;
    static constexpr int STAGES = BUDGET / STAGE_BYTES;
    static constexpr int BLOCKS_PER_SM = BT <= 64 ? 2 : 1;
    static constexpr int TMEM_COLS = BT < 32 ? 32 : BT;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

// ------------------------------------------------------------------------------------------
// The kernel.  grid = (row tiles of W, token tiles, splits of K)
// ------------------------------------------------------------------------------------------
template <int BT>
__global__ void __launch_bounds__(TC_THREADS, TcConfig<BT>::BLOCKS_PER_SM)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                    void* __restrict__ C, int c_dtype, long ldc, int M, int N, int K, int kblocks_per_split,
                    int epilogue, int* __restrict__ status, TcWaits waits) {
    using Cfg = TcConfig<BT>;
    const uint32_t spin_limit = waits.spin_limit;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty = full + Cfg::STAGES;
    uint64_t* tmem_full = empty + Cfg::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
    int* s_flag = reinterpret_cast<int*>(tmem_slot + 1);      // [0] error seen, [1] this block reduces the splits

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TC_ROWS;
    const int m0 = blockIdx.y * BT;
    const int total_kblocks = (K + TC_BK - 1) / TC_BK;
    const int kb_beg = blockIdx.z * kblocks_per_split;
    const int kb_end = min(total_kblocks, kb_beg + kblocks_per_split);
    const int n_kb = max(0, kb_end - kb_beg);
    const int ksplit = gridDim.z;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(tmem_full, 1);
        s_flag[0] = 0;
        s_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    float c_pre[4] = {0.0f, 0.0f, 0.0f, 0.0f};                            // epilogue threads: see there

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            // W does not depend on the kernel before this one: the ring fills with W tiles before the
            // wait for that kernel (programmatic dependent launch), the A tiles follow after it
            const int early = waits.hold_producer ? 0 : (n_kb < Cfg::STAGES ? n_kb : Cfg::STAGES);
            pdl_trigger();
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(&full[i], Cfg::STAGE_BYTES);
                tma_load_2d(smem + (size_t)i * Cfg::STAGE_BYTES, &map_w, (kb_beg + i) * TC_BK, n0, &full[i]);
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(smem + (size_t)i * Cfg::STAGE_BYTES + TC_ROWS * TC_BK * 2, &map_a, (kb_beg + i) * TC_BK, m0, &full[i]);
            for (int i = early; i < n_kb && !waits.hold_producer; ++i) {
                const int s = i % Cfg::STAGES;
                const uint32_t phase = (i / Cfg::STAGES) & 1;
                if (!MBAR_WAIT(&empty[s], phase ^ 1)) {
                    atomicOr(status, BFI_STATUS_TIMEOUT);
                    s_flag[0] = 1;
                    break;
                }
                unsigned char* stage = smem + (size_t)s * Cfg::STAGE_BYTES;
                mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
                const int k = (kb_beg + i) * TC_BK;
                tma_load_2d(stage, &map_w, k, n0, &full[s]);
                tma_load_2d(stage + TC_ROWS * TC_BK * 2, &map_a, k, m0, &full[s]);
            }
        } else {
            pdl_trigger();
            pdl_wait();
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(TC_ROWS, BT);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % Cfg::STAGES;
                const uint32_t phase = (i / Cfg::STAGES) & 1;
                if (!MBAR_WAIT(&full[s], phase)) {
                    atomicOr(status, BFI_STATUS_TIMEOUT);
                    s_flag[0] = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t wa = smem_u32(smem + (size_t)s * Cfg::STAGE_BYTES);
                const uint32_t aa = wa + TC_ROWS * TC_BK * 2;
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)
                    umma_bf16(tmem_base, umma_desc_sw128(wa + kk * 32), umma_desc_sw128(aa + kk * 32), idesc,
                              (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&empty[s]);          // the stage is free once these MMAs have read it
            }
            umma_commit(tmem_full);               // arrives when every MMA issued above has completed
        }
    } else {
        // ---------------- epilogue warps: TMEM lanes 32*(warp % 4) .. +31
        pdl_trigger();
        pdl_wait();                                      // C may still be in use by the kernel before
        const int quad = warp & 3;
        const int n_local = quad * 32 + lane;
        const int n = n0 + n_local;
        bool ok = true;
        if (ksplit > 1 && epilogue == EPI_ACCUMULATE && n < N) {
            // the values this thread will add to (no kernel in flight writes them any more) are
            // fetched now, while the products run, instead of behind them
            const int per_rank = (BT + ksplit - 1) / ksplit;
            const int j0 = (int)blockIdx.z * per_rank;
            const float* c_in = reinterpret_cast<const float*>(C);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (u < per_rank && j0 + u < BT && m0 + j0 + u < M) c_pre[u] = c_in[(size_t)(m0 + j0 + u) * ldc + n];
        }
        if (n_kb > 0) {
            ok = MBAR_WAIT(tmem_full, 0);
            if (!ok && lane == 0) {
                atomicOr(status, BFI_STATUS_TIMEOUT);
                s_flag[0] = 1;
            }
        }
        tc_fence_after();
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);

        if (ksplit > 1) {
            // partial tile -> this block's shared memory as [token][row] (the ring is idle by now)
            float* part = reinterpret_cast<float*>(smem);
#pragma unroll 1
            for (int c = 0; c < BT / 16; ++c) {
                float v[16];
                if (ok && n_kb > 0) {
                    tmem_ld16(lane_addr + c * 16, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) part[(c * 16 + j) * TC_ROWS + n_local] = v[j];
            }
        } else if (ok) {
            // 16 tokens at a time.  All of a chunk's values are computed (and, when adding, all the old
            // values fetched) before the first store, without a branch between them: one warp per
            // scheduler has nothing else to cover the latency of a shuffle, an exponential or a load.
#pragma unroll 1
            for (int c = 0; c < BT / 16; ++c) {
                const int m_c = m0 + c * 16;
                if (m_c >= M) break;
                const int rows_here = min(16, M - m_c);
                float v[16];
                tmem_ld16(lane_addr + c * 16, v);
                if (epilogue == EPI_SWIGLU) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = silu_mul_tc(v[j], __shfl_down_sync(0xffffffffu, v[j], 1));
                    if ((lane & 1) == 0 && n + 1 < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < rows_here) store_from_f32(C, c_dtype, (size_t)(m_c + j) * ldc + (n >> 1), v[j]);
                    }
                } else if (n < N) {
                    if (epilogue == EPI_ACCUMULATE) {
                        float* c_io = reinterpret_cast<float*>(C) + (size_t)m_c * ldc + n;
                        float old[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) old[j] = j < rows_here ? c_io[(size_t)j * ldc] : 0.0f;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < rows_here) c_io[(size_t)j * ldc] = old[j] + v[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < rows_here) store_from_f32(C, c_dtype, (size_t)(m_c + j) * ldc + n, v[j]);
                    }
                }
            }
        }
    }

    // ---------------- split K: the cluster's blocks add their partial tiles
    if (ksplit > 1) {
        __syncwarp();
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp >= 2) {
            const int quad = warp & 3;
            const int n_local = quad * 32 + lane;
            const int n = n0 + n_local;
            const int rank = blockIdx.z;                         // cluster dims are (1, 1, ksplit)
            const int per_rank = (BT + ksplit - 1) / ksplit;     // tokens this block finishes
            // the same offset in every block's shared memory (at most 8 blocks in a cluster)
            uint32_t remote[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const uint32_t local = smem_u32(smem);
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote[r]) : "r"(local), "r"(r < ksplit ? r : 0));
            }
            // four tokens at a time: every split's partial value of all four (and, when adding, the old
            // values beyond the four fetched before the products) is asked for before the first is
            // used, then each token's sum is taken in split order
            const int j_beg = rank * per_rank;
            const int j_end = min(min(BT, (rank + 1) * per_rank), M - m0);
#pragma unroll 1
            for (int j0 = j_beg; j0 < j_end; j0 += 4) {
                float x[4][8], old[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const bool live = j0 + u < j_end;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        x[u][r] = 0.0f;
                        if (live && r < ksplit)
                            asm volatile("ld.shared::cluster.f32 %0, [%1];"
                                         : "=f"(x[u][r])
                                         : "r"(remote[r] + (uint32_t)((j0 + u) * TC_ROWS + n_local) * 4));
                    }
                    old[u] = c_pre[u];
                    if (epilogue == EPI_ACCUMULATE && j0 > j_beg && live && n < N)
                        old[u] = reinterpret_cast<const float*>(C)[(size_t)(m0 + j0 + u) * ldc + n];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const bool live = j0 + u < j_end;                // the same for the whole warp
                    const int m = m0 + j0 + u;
                    float v = 0.0f;
#pragma unroll
                    for (int r = 0; r < 8; ++r) v += x[u][r];
                    if (epilogue == EPI_SWIGLU) {
                        const float act = silu_mul_tc(v, __shfl_down_sync(0xffffffffu, v, 1));
                        if (live && (lane & 1) == 0 && n + 1 < N) store_from_f32(C, c_dtype, (size_t)m * ldc + (n >> 1), act);
                    } else if (live && n < N) {
                        const size_t o = (size_t)m * ldc + n;
                        if (epilogue == EPI_ACCUMULATE)
                            reinterpret_cast<float*>(C)[o] = old[u] + v;
                        else
                            store_from_f32(C, c_dtype, o, v);
                    }
                }
            }
        }
        // no block may leave while another still reads its shared memory
        __syncwarp();
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }

    // ---------------- common tail: everyone meets, copies in flight are drained, TMEM is freed
    tc_fence_before();
    __syncthreads();
    if (s_flag[0] && warp == 0 && lane == 0) {
        // a wait ran out: let outstanding TMA writes land (bounded) before the block's memory is reused
        for (int s = 0; s < Cfg::STAGES && s < n_kb; ++s) {
            const int last = ((n_kb - 1 - s) / Cfg::STAGES) * Cfg::STAGES + s;   // last k block that used stage s
            MBAR_WAIT(&full[s], (uint32_t)((last / Cfg::STAGES) & 1));
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
    BFI_TRACE_END();
}

// ------------------------------------------------------------------------------------------
// Many tokens (prompts): tokens on the lanes.  D[128 tokens, tile_n features] per tile, so a thread
// holds consecutive features of one token after tcgen05.ld (SiLU*mul pairs sit in one thread); they
// leave through a staging tile in shared memory, as whole rows (tp_emit_group), or, where a group
// is not whole, straight from the registers as 16-byte words.  The kernel is persistent: each block walks over
// tiles, and the two halves of tensor memory (2 x 256 columns) alternate as accumulators, so the
// epilogue of one tile runs while the tensor cores work on the next.  tile_n (a multiple of 16, at
// most 256) is chosen per product so that the tiles fill whole rounds of the SMs: 2560 features
// x 2048 tokens are 160 tiles of 256 (two rounds, the second almost empty) but 288 tiles of 144.
//   barriers: full/empty per ring stage, tmem_full/tmem_empty per accumulator
// ------------------------------------------------------------------------------------------
#define TP_TOKENS 128
#define TP_FEATS 256                                             // widest tile; the accumulators' stride
#define TP_RING_BYTES (4 * (TP_TOKENS + TP_FEATS) * TC_BK * 2)   // 192 KB
#define TP_MAX_STAGES 8
#define TP_EPI_WARPS 8                                           // two per quarter of the TMEM lanes: each takes half a tile's features
#define TP_THREADS (64 + 32 * TP_EPI_WARPS)
#define TP_STAGE_BYTES 4096                                      // per epilogue warp: 32 token rows of 128 bytes on their way out
#define TP_SMEM ((size_t)TP_RING_BYTES + 1024 + 256 + TP_EPI_WARPS * TP_STAGE_BYTES)

// A group of G chunks (16 features each) of an epilogue warp's 32 tokens, out through shared memory.
// After tcgen05.ld a lane holds ONE token's values, so a store straight from the registers touches 32
// different lines with a few bytes each; here each lane leaves its token's row (up to 128 bytes, as
// 16-byte pieces, piece j at position j ^ (row & 7): no bank conflicts either way) in the warp's
// staging tile, and the warp then writes (or, adding, reads and writes) whole rows: 8 lanes a row.
// G = 2 for float32 outputs, 4 for bfloat16 and for the gated epilogue.
template <int G>
__device__ __forceinline__ void tp_emit_group(uint4* stage, const float (&v)[G][16], int lane, int epilogue, int c_dtype,
                                              void* __restrict__ C, long ldc, int m_base, int M, int n0) {
    uint4 piece[8];
    int n_pieces;
    size_t out_byte0;                     // of the group's first output in its row of C
    if (epilogue == EPI_SWIGLU) {
        if (c_dtype == BFI_BF16) {        // 16 features -> 8 outputs -> one piece per chunk
            n_pieces = G;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                uint32_t pk[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(silu_mul_tc(v[g][4 * j], v[g][4 * j + 1]),
                                                              silu_mul_tc(v[g][4 * j + 2], v[g][4 * j + 3]));
                    pk[j] = *reinterpret_cast<uint32_t*>(&t2);
                }
                piece[g] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
            out_byte0 = (size_t)(n0 >> 1) * 2;
        } else {                          // float32: two pieces per chunk
            n_pieces = 2 * G;
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    piece[(2 * g + q) & 7] = make_uint4(__float_as_uint(silu_mul_tc(v[g][8 * q], v[g][8 * q + 1])),
                                                        __float_as_uint(silu_mul_tc(v[g][8 * q + 2], v[g][8 * q + 3])),
                                                        __float_as_uint(silu_mul_tc(v[g][8 * q + 4], v[g][8 * q + 5])),
                                                        __float_as_uint(silu_mul_tc(v[g][8 * q + 6], v[g][8 * q + 7])));
            out_byte0 = (size_t)(n0 >> 1) * 4;
        }
    } else if (c_dtype == BFI_BF16) {     // two pieces per chunk
        n_pieces = 2 * G;
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t pk[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 t2 = __floats2bfloat162_rn(v[g][8 * q + 2 * j], v[g][8 * q + 2 * j + 1]);
                    pk[j] = *reinterpret_cast<uint32_t*>(&t2);
                }
                piece[(2 * g + q) & 7] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        out_byte0 = (size_t)n0 * 2;
    } else {                              // float32, stored or added: four pieces per chunk (G = 2)
        n_pieces = 4 * G;
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int q = 0; q < 4; ++q)
                piece[(4 * g + q) & 7] = make_uint4(__float_as_uint(v[g][4 * q]), __float_as_uint(v[g][4 * q + 1]),
                                                    __float_as_uint(v[g][4 * q + 2]), __float_as_uint(v[g][4 * q + 3]));
        out_byte0 = (size_t)n0 * 4;
    }
    __syncwarp();                         // the tile is free: every lane has read what the group before left
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (j < n_pieces) stage[lane * 8 + (j ^ (lane & 7))] = piece[j];
    __syncwarp();
    const size_t row_bytes = (size_t)ldc * (c_dtype == BFI_F32 ? 4 : 2);
    const int shift = n_pieces == 8 ? 3 : (n_pieces == 4 ? 2 : 1);       // rows per pass: 32 >> shift lanes... pieces a row = 1 << shift
    unsigned char* c_bytes = reinterpret_cast<unsigned char*>(C);
    if (epilogue == EPI_ACCUMULATE) {
        float4 old[8];
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int idx = it * 32 + lane, row = idx >> 3, j = idx & 7;
            old[it] = m_base + row < M ? __ldcg(reinterpret_cast<const float4*>(c_bytes + (size_t)(m_base + row) * row_bytes + out_byte0 + j * 16))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int idx = it * 32 + lane, row = idx >> 3, j = idx & 7;
            const uint4 add = stage[row * 8 + (j ^ (row & 7))];
            if (m_base + row < M)
                *reinterpret_cast<float4*>(c_bytes + (size_t)(m_base + row) * row_bytes + out_byte0 + j * 16) =
                    make_float4(old[it].x + __uint_as_float(add.x), old[it].y + __uint_as_float(add.y),
                                old[it].z + __uint_as_float(add.z), old[it].w + __uint_as_float(add.w));
        }
    } else {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            if (it >= n_pieces) break;
            const int idx = it * 32 + lane, row = idx >> shift, j = idx & (n_pieces - 1);
            if (m_base + row < M)
                *reinterpret_cast<uint4*>(c_bytes + (size_t)(m_base + row) * row_bytes + out_byte0 + j * 16) =
                    stage[row * 8 + (j ^ (row & 7))];
        }
    }
}


template <int HALVES>
__global__ void __launch_bounds__(TP_THREADS, 1)
gemm_tcgen05_prefill_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                            void* __restrict__ C, int c_dtype, long ldc, int M, int N, int K, int tiles_m, int tiles_n,
                            int tile_n, int n_stages, int epilogue, int vec_ok, int* __restrict__ status, TcWaits waits) {
    const uint32_t spin_limit = waits.spin_limit;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)TP_RING_BYTES);
    uint64_t* empty = full + TP_MAX_STAGES;
    uint64_t* tmem_full = empty + TP_MAX_STAGES;  // [2]
    constexpr int TILE_TOKENS = HALVES * TP_TOKENS;
    const uint32_t stage_bytes = (uint32_t)(TILE_TOKENS + tile_n) * TC_BK * 2;  // a multiple of 2048
    uint64_t* tmem_empty = tmem_full + 2;         // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    int* s_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (K + TC_BK - 1) / TC_BK;
    const int n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], TP_EPI_WARPS);   // one arrival per epilogue warp
        }
        s_flag[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();                                 // the kernel after this one may start its own preamble

    // tiles in bands of 8 token tiles: blocks that run together share W tiles and A tiles in L2
    auto tile_coords = [&](int tile, int& tm, int& tn) {
        const int band = 8;
        const int per_band = band * tiles_n;
        const int b = tile / per_band, r = tile - b * per_band;
        const int rows_here = min(band, tiles_m - b * band);
        tn = r / rows_here;
        tm = b * band + (r - tn * rows_here);
    };

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                            // k blocks issued so far, over all tiles
            bool first = true;
            for (int tile = blockIdx.x; tile < n_tiles && !s_flag[0] && !waits.hold_producer; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, tm, tn);
                int i0 = 0;
                if (first) {
                    // W does not depend on the kernel before this one: the first stages' W halves travel
                    // before the wait for that kernel, their A halves after it
                    const int early = n_kb < n_stages ? n_kb : n_stages;
                    for (int i = 0; i < early; ++i) {
                        mbar_expect_tx(&full[i], stage_bytes);
                        tma_load_2d(smem + (size_t)i * stage_bytes + TILE_TOKENS * TC_BK * 2, &map_w, i * TC_BK, tn * tile_n,
                                    &full[i]);
                    }
                    pdl_wait();
                    for (int i = 0; i < early; ++i)
                        tma_load_2d(smem + (size_t)i * stage_bytes, &map_a, i * TC_BK, tm * TILE_TOKENS, &full[i]);
                    it = i0 = early;
                    first = false;
                }
                for (int i = i0; i < n_kb; ++i, ++it) {
                    const int s = it % n_stages;
                    const uint32_t phase = (it / n_stages) & 1;
                    if (it >= n_stages && !MBAR_WAIT(&empty[s], phase ^ 1)) {
                        atomicOr(status, BFI_STATUS_TIMEOUT);
                        s_flag[0] = 1;
                        break;
                    }
                    unsigned char* stage = smem + (size_t)s * stage_bytes;
                    mbar_expect_tx(&full[s], stage_bytes);
                    tma_load_2d(stage, &map_a, i * TC_BK, tm * TILE_TOKENS, &full[s]);
                    tma_load_2d(stage + TILE_TOKENS * TC_BK * 2, &map_w, i * TC_BK, tn * tile_n, &full[s]);
                }
            }
            if (first) pdl_wait();
        } else {
            pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(TP_TOKENS, tile_n);
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !s_flag[0]; tile += gridDim.x, ++local) {
                // HALVES == 1: the two accumulators alternate between tiles.  HALVES == 2: a tile's two
                // token halves own one accumulator each, and a half may be overwritten as soon as the
                // epilogue has drained it.
                const int acc = local & 1;
                bool ok = true;
                if (HALVES == 1 && local >= 2 && !MBAR_WAIT(&tmem_empty[acc], (((uint32_t)(local >> 1)) & 1) ^ 1)) ok = false;
                tc_fence_after();
                for (int i = 0; ok && i < n_kb; ++i, ++it) {
                    const int s = it % n_stages;
                    const uint32_t phase = (it / n_stages) & 1;
                    if (!MBAR_WAIT(&full[s], phase)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t aa = smem_u32(smem + (size_t)s * stage_bytes);
                    const uint32_t wa = aa + TILE_TOKENS * TC_BK * 2;
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) {
                        if (HALVES == 2 && i == 0 && local >= 1) {
                            if (!MBAR_WAIT(&tmem_empty[h], (uint32_t)((local - 1) & 1))) {
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                        }
                        const uint32_t d_addr = tmem_base + (uint32_t)(HALVES == 1 ? acc : h) * TP_FEATS;
                        const uint32_t ah = aa + h * TP_TOKENS * TC_BK * 2;
#pragma unroll
                        for (int kk = 0; kk < TC_BK / 16; ++kk)
                            umma_bf16(d_addr, umma_desc_sw128(ah + kk * 32), umma_desc_sw128(wa + kk * 32), idesc,
                                      (i > 0 || kk > 0) ? 1u : 0u);
                    }
                    if (!ok) break;
                    umma_commit(&empty[s]);
                }
                umma_commit(&tmem_full[HALVES == 1 ? acc : 0]);
                if (!ok) {
                    atomicOr(status, BFI_STATUS_TIMEOUT);
                    s_flag[0] = 1;
                    break;
                }
            }
        }
    } else {
        pdl_wait();                                      // C may still be in use by the kernel before
        const int quad = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            int tm, tn;
            tile_coords(tile, tm, tn);
            const int full_idx = HALVES == 1 ? (local & 1) : 0;
            const uint32_t full_parity = HALVES == 1 ? (uint32_t)((local >> 1) & 1) : (uint32_t)(local & 1);
            if (epilogue == EPI_ACCUMULATE) {
                // the sums this tile will be added to are asked into L2 now, while its products run:
                // in a step the residual has long left L2 when a product comes to add into it
                const int n_first = tn * tile_n;
                const int n_feats = min(tile_n, N - n_first);
                for (int h = 0; h < HALVES; ++h) {
                    const int mm = tm * TILE_TOKENS + h * TP_TOKENS + quad * 32 + lane;
                    if (mm < M) {
                        const char* row = reinterpret_cast<const char*>(C) + ((size_t)mm * ldc + n_first) * 4;
                        for (int off = (warp - 2 < 4 ? 0 : 128); off < n_feats * 4; off += 256)
                            asm volatile("prefetch.global.L2 [%0];" ::"l"(row + off));
                    }
                }
            }
            if (!MBAR_WAIT(&tmem_full[full_idx], full_parity)) {
                if (lane == 0) {
                    atomicOr(status, BFI_STATUS_TIMEOUT);
                    s_flag[0] = 1;
                }
                break;
            }
            tc_fence_after();
            for (int h = 0; h < HALVES; ++h) {
            const int acc = HALVES == 1 ? (local & 1) : h;
            const int m = tm * TILE_TOKENS + h * TP_TOKENS + quad * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * TP_FEATS;
            // the two warps of a lane quarter share a token's features: chunks of 16, the first half and the second
            const int n_chunks = tile_n / 16;
            const int c_beg = (warp - 2) < 4 ? 0 : (n_chunks + 1) / 2;
            const int c_end = (warp - 2) < 4 ? (n_chunks + 1) / 2 : n_chunks;
            // whole groups of chunks go out through the warp's staging tile, what is left (a ragged
            // edge of N, rows of C that are not 16-byte aligned, a last odd chunk) straight from the registers
            int c_direct = c_beg;
            if (vec_ok) {
                uint4* stage = reinterpret_cast<uint4*>(smem + TP_RING_BYTES + 256) + (warp - 2) * (TP_STAGE_BYTES / 16);
                const int m_base = tm * TILE_TOKENS + h * TP_TOKENS + quad * 32;
                const bool wide = !(epilogue == EPI_SWIGLU || c_dtype == BFI_BF16);      // float32 rows: 2 chunks are 128 bytes
#pragma unroll 1
                while (c_direct < c_end) {
                    const int n0 = tn * tile_n + c_direct * 16;
                    if (!wide && c_direct + 4 <= c_end && n0 + 64 <= N) {
                        float v[4][16];
                        tmem_ld64(taddr + c_direct * 16, v);
                        tp_emit_group<4>(stage, v, lane, epilogue, c_dtype, C, ldc, m_base, M, n0);
                        c_direct += 4;
                    } else if (c_direct + 2 <= c_end && n0 + 32 <= N) {
                        float v[2][16];
                        tmem_ld32(taddr + c_direct * 16, v);
                        tp_emit_group<2>(stage, v, lane, epilogue, c_dtype, C, ldc, m_base, M, n0);
                        c_direct += 2;
                    } else {
                        break;
                    }
                }
            }
#pragma unroll 1
            for (int c = c_direct; c < c_end; ++c) {
                const int n = tn * tile_n + c * 16;
                if (n >= N) break;
                float v[16];
                tmem_ld16(taddr + c * 16, v);
                if (m >= M) continue;
                const bool whole = vec_ok && n + 16 <= N;
                if (epilogue == EPI_SWIGLU) {
                    if (whole) {
                        uint32_t pk[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            pk[j] = c_dtype == BFI_BF16
                                        ? ([&] {
                                              __nv_bfloat162 t2 = __floats2bfloat162_rn(silu_mul_tc(v[4 * j], v[4 * j + 1]),
                                                                                        silu_mul_tc(v[4 * j + 2], v[4 * j + 3]));
                                              return *reinterpret_cast<uint32_t*>(&t2);
                                          })()
                                        : 0u;
                        if (c_dtype == BFI_BF16) {
                            *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(C) + (size_t)m * ldc + (n >> 1)) =
                                make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        } else {
                            float* o = reinterpret_cast<float*>(C) + (size_t)m * ldc + (n >> 1);
#pragma unroll
                            for (int j = 0; j < 8; ++j) o[j] = silu_mul_tc(v[2 * j], v[2 * j + 1]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j += 2)
                            if (n + j + 1 < N)
                                store_from_f32(C, c_dtype, (size_t)m * ldc + ((n + j) >> 1), silu_mul_tc(v[j], v[j + 1]));
                    }
                } else if (epilogue == EPI_ACCUMULATE) {
                    float* o = reinterpret_cast<float*>(C) + (size_t)m * ldc + n;
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float4 x = *reinterpret_cast<float4*>(o + 4 * j);
                            x.x += v[4 * j];
                            x.y += v[4 * j + 1];
                            x.z += v[4 * j + 2];
                            x.w += v[4 * j + 3];
                            *reinterpret_cast<float4*>(o + 4 * j) = x;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n + j < N) o[j] += v[j];
                    }
                } else if (whole && c_dtype == BFI_BF16) {
                    uint32_t pk[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        __nv_bfloat162 t2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                        pk[j] = *reinterpret_cast<uint32_t*>(&t2);
                    }
                    uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(C) + (size_t)m * ldc + n);
                    o[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    o[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                } else if (whole) {
                    float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(C) + (size_t)m * ldc + n);
#pragma unroll
                    for (int j = 0; j < 4; ++j) o[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (n + j < N) store_from_f32(C, c_dtype, (size_t)m * ldc + n + j, v[j]);
                }
            }
            // this warp is done with the accumulator: the tensor cores may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (s_flag[0] && warp == 0 && lane == 0) {
        // a wait ran out: give outstanding TMA writes a bounded time to land
        for (int s = 0; s < n_stages; ++s) MBAR_WAIT(&full[s], 0), MBAR_WAIT(&full[s], 1);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    BFI_TRACE_END();
}

// ------------------------------------------------------------------------------------------
// Host side: tensor maps (cached), planning, launch
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

struct MapKey {
    const void* ptr;
    long rows, cols, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        h = h * 1000003u ^ std::hash<long>()(k.rows);
        h = h * 1000003u ^ std::hash<long>()(k.cols);
        h = h * 1000003u ^ std::hash<long>()(k.ld);
        return h * 1000003u ^ std::hash<int>()(k.box_rows);
    }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
static std::mutex g_maps_mutex;

int bfi_tensor_map_bf16(const void* ptr, long rows, long cols, long ld, int box_rows, CUtensorMap* out) {
    MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
        *out = it->second;
        return 0;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return bfi_fail("gemm_tcgen05: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return bfi_fail("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps[key] = m;
    *out = m;
    return 0;
}

struct TcPlan {
    int bt, tiles_n, tiles_m, ksplit, kblocks_per_split;
};

// Overrides of the planners' choices, for tests and experiments.  An override holds for ONE call of
// bfi_gemm_tcgen05_bf16 (the next one, which takes it and clears it, whether or not it launches), so
// nothing a test sets can outlive that test.  0 keeps the built-in choice.
struct TcTune {
    int ksplit;      // few-row kernel: splits of K
    int tile_n;      // many-row kernel: features per tile
    int halves;      // many-row kernel: one or two halves of 128 tokens
};
static TcTune g_tc_tune = {0, 0, 0};
static TcTune take_tc_tune() {
    const TcTune t = g_tc_tune;
    g_tc_tune = TcTune{0, 0, 0};
    return t;
}
extern "C" int bfi_gemm_tcgen05_tune_next(int ksplit, int tile_n, int halves) {
    g_tc_tune.ksplit = ksplit > 0 ? ksplit : 0;
    g_tc_tune.tile_n = (tile_n >= 16 && tile_n <= TP_FEATS && tile_n % 16 == 0) ? tile_n : 0;
    g_tc_tune.halves = (halves == 1 || halves == 2) ? halves : 0;
    return 0;
}

static TcPlan plan_tc(int M, int N, int K, int g_tc_tune_ksplit) {
    const bool allow_split = true;
    TcPlan p;
    p.bt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
    p.tiles_n = (N + TC_ROWS - 1) / TC_ROWS;
    p.tiles_m = (M + p.bt - 1) / p.bt;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    p.ksplit = 1;
    const long tiles = (long)p.tiles_n * p.tiles_m;
    const long slots = (p.bt <= 64 ? 2L : 1L) * bfi_sm_count();     // blocks resident at once
    if (allow_split && tiles * 2 <= slots) {
        // few tiles: split K so that the grid fills the resident slots in one wave, with at least
        // 8 k blocks per split (shorter runs cost more in fill and reduction than they gain)
        int want = (int)(slots / tiles);
        if (want > 8) want = 8;                         // portable cluster size
        while (want > 1 && kblocks / want < 8) --want;
        p.ksplit = want;
    }
    if (g_tc_tune_ksplit > 0) p.ksplit = g_tc_tune_ksplit > 8 ? 8 : g_tc_tune_ksplit;
    p.kblocks_per_split = (kblocks + p.ksplit - 1) / p.ksplit;
    p.ksplit = (kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split;   // no empty splits
    return p;
}

template <int BT>
static int launch_tc(const TcPlan& p, const CUtensorMap& mw, const CUtensorMap& ma, void* C, int c_dtype, long ldc,
                     int M, int N, int K, int epilogue, int* status, cudaStream_t stream, TcWaits waits) {
    using Cfg = TcConfig<BT>;
    auto kernel = gemm_tcgen05_kernel<BT>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);
        if (e != cudaSuccess)
            return bfi_fail("gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e));
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.tiles_n, p.tiles_m, p.ksplit);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (p.ksplit > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = p.ksplit;
        ++n_attr;
    }
    if (g_bfi_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mw, ma, C, c_dtype, ldc, M, N, K, p.kblocks_per_split, epilogue, status, waits);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return bfi_fail("gemm_tcgen05: launch failed: %s", cudaGetErrorString(e));
    }
    return bfi_check_launch("gemm_tcgen05");
}

static int launch_tc_prefill(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype, long ldc, int M,
                             int N, int K, int epilogue, int* status, cudaStream_t stream, TcWaits waits, TcTune tune) {
    const int g_tp_tune_tile_n = tune.tile_n, g_tp_tune_halves = tune.halves;
    static bool configured = false;
    const int n_sm = bfi_sm_count();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_prefill_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)TP_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_tcgen05_prefill_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TP_SMEM);
        if (e != cudaSuccess)
            return bfi_fail("gemm_tcgen05: cannot reserve %zu bytes of shared memory: %s", (size_t)TP_SMEM, cudaGetErrorString(e));
        configured = true;
    }
    // The tile (one or two halves of 128 tokens x tile_n features) that takes the least time by an
    // estimate fitted to measurements: rounds over the SMs x (k blocks x the time of a k block, which
    // grows slowly with the width and is 1.4 x longer for two halves, + a tile's share that no other
    // tile hides: little when the accumulators alternate, the whole epilogue when a tile owns both).
    int halves = 1, tile_n = TP_FEATS;
    {
        const double n_kb = (double)((K + TC_BK - 1) / TC_BK);
        double best = -1.0;
        for (int h = 1; h <= (M > TP_TOKENS ? 2 : 1); ++h) {
            if (g_tp_tune_halves && h != g_tp_tune_halves) continue;
            for (int tn = TP_FEATS; tn >= 128; tn -= 16) {
                if (g_tp_tune_tile_n && tn != g_tp_tune_tile_n) continue;
                const long t = (long)((M + h * TP_TOKENS - 1) / (h * TP_TOKENS)) * ((N + tn - 1) / tn);
                const double kb_time = (h == 1 ? 0.351 : 0.507) + 0.00048 * tn;
                const double cost = (double)((t + n_sm - 1) / n_sm) * (n_kb * kb_time + (h == 1 ? 2.0 : 10.0));
                if (best < 0.0 || cost < best) {
                    best = cost;
                    halves = h;
                    tile_n = tn;
                }
            }
        }
        if (best < 0.0) {               // a forced width below 128
            tile_n = g_tp_tune_tile_n;
            halves = g_tp_tune_halves ? g_tp_tune_halves : 1;
        }
    }
    const int tile_tokens = halves * TP_TOKENS;
    const int tiles_m = (M + tile_tokens - 1) / tile_tokens, tiles_n = (N + tile_n - 1) / tile_n;
    const long tiles = (long)tiles_m * tiles_n;
    const int grid = (int)(tiles < n_sm ? tiles : n_sm);
    const int stage_bytes = (tile_tokens + tile_n) * TC_BK * 2;
    int n_stages = TP_RING_BYTES / stage_bytes;
    if (n_stages > TP_MAX_STAGES) n_stages = TP_MAX_STAGES;
    CUtensorMap ma, mw;
    int rc = bfi_tensor_map_bf16(A, M, K, lda, tile_tokens, &ma);
    if (rc) return rc;
    rc = bfi_tensor_map_bf16(W, N, K, ldw, tile_n, &mw);
    if (rc) return rc;
    // whole 16-byte stores need aligned rows: output row stride and base
    const int elem = dtype_size(c_dtype);
    const int vec_ok = ((ldc * elem) % 16 == 0 && ((uintptr_t)C & 15) == 0) ? 1 : 0;
    if (halves == 2)
        bfi_launch(gemm_tcgen05_prefill_kernel<2>, dim3(grid), dim3(TP_THREADS), TP_SMEM, stream, ma, mw, C, c_dtype, ldc, M, N,
                   K, tiles_m, tiles_n, tile_n, n_stages, epilogue, vec_ok, status, waits);
    else
        bfi_launch(gemm_tcgen05_prefill_kernel<1>, dim3(grid), dim3(TP_THREADS), TP_SMEM, stream, ma, mw, C, c_dtype, ldc, M, N,
                   K, tiles_m, tiles_n, tile_n, n_stages, epilogue, vec_ok, status, waits);
    return bfi_check_launch("gemm_tcgen05_prefill");
}

static int gemm_tcgen05_launch(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype, long ldc, int M,
                               int N, int K, int epilogue, int* status, cudaStream_t stream, TcWaits waits) {
    BFI_REQUIRE(dtype_ok(c_dtype), "gemm_tcgen05: unknown output dtype code %d", c_dtype);
    BFI_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
    BFI_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tcgen05: unknown epilogue %d", epilogue);
    BFI_REQUIRE(status != nullptr, "gemm_tcgen05: a status word is required");
    if (epilogue == EPI_ACCUMULATE) BFI_REQUIRE(c_dtype == BFI_F32, "gemm_tcgen05: accumulation needs a float32 output");
    if (epilogue == EPI_SWIGLU) BFI_REQUIRE(N % 2 == 0, "gemm_tcgen05: the gated epilogue needs an even N, got %d", N);
    const TcTune tune = take_tc_tune();
    if (M == 0) return 0;
    // TMA: 16-byte aligned bases and row strides
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15)) return 2;
    if (M >= 128) return launch_tc_prefill(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, status, stream, waits, tune);
    TcPlan p = plan_tc(M, N, K, tune.ksplit);
    if (p.tiles_m > 65535) return 2;
    CUtensorMap mw, ma;
    int rc = bfi_tensor_map_bf16(W, N, K, ldw, TC_ROWS, &mw);
    if (rc) return rc;
    rc = bfi_tensor_map_bf16(A, M, K, lda, p.bt, &ma);
    if (rc) return rc;
    switch (p.bt) {
        case 16: return launch_tc<16>(p, mw, ma, C, c_dtype, ldc, M, N, K, epilogue, status, stream, waits);
        case 32: return launch_tc<32>(p, mw, ma, C, c_dtype, ldc, M, N, K, epilogue, status, stream, waits);
        case 64: return launch_tc<64>(p, mw, ma, C, c_dtype, ldc, M, N, K, epilogue, status, stream, waits);
        case 128: return launch_tc<128>(p, mw, ma, C, c_dtype, ldc, M, N, K, epilogue, status, stream, waits);
        default: return launch_tc<256>(p, mw, ma, C, c_dtype, ldc, M, N, K, epilogue, status, stream, waits);
    }
}

// Returns 0 on success, 1 on error, 2 when the shape is not taken (nothing launched).
// `status` receives BFI_STATUS_TIMEOUT (8) if a bounded wait inside the kernel ran out.
extern "C" int bfi_gemm_tcgen05_bf16(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype, long ldc,
                                     int M, int N, int K, int epilogue, int* status, cudaStream_t stream) {
    return gemm_tcgen05_launch(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, status, stream, tc_waits_default());
}

// For the tests of the time-out path: the same launch, but every bounded wait gives up after
// `spin_limit` polls (at most 65536 here, so the launch ends within milliseconds) and, with
// hold_producer != 0, the thread that issues the TMA copies issues none.  The consumers' waits then
// run out by construction: the launch records BFI_STATUS_TIMEOUT in `status`, gives its copies (there
// are none) a bounded time to land, frees its tensor memory and returns; C holds nothing of use.
// No fault, no trap and no unbounded wait is involved.
extern "C" int bfi_gemm_tcgen05_bf16_wait_probe(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype,
                                                long ldc, int M, int N, int K, int epilogue, int* status,
                                                unsigned spin_limit, int hold_producer, cudaStream_t stream) {
    BFI_REQUIRE(spin_limit >= 1 && spin_limit <= 65536, "gemm_tcgen05 wait probe: spin limit %u outside 1..65536", spin_limit);
    return gemm_tcgen05_launch(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, status, stream,
                               TcWaits{spin_limit, hold_producer ? 1 : 0});
}

BFI_TRACE_EXPORT(gemm_tcgen05)
