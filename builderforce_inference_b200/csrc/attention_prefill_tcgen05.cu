// Prompt attention for bfloat16 on the fifth-generation tensor cores: every new token of a step
// attends causally over the cached keys and values of its sequence (the step's own tokens are
// already in the cache), with an optional window (crates/bfi-core/src/cpu.rs:328-392).
//
// One block per (sequence, query head, 128 consecutive tokens).  Keys and values arrive as tiles
// of 128 positions (two cache pages) by TMA with the 128-byte swizzle; both products run as
// tcgen05.mma with float32 accumulators in tensor memory:
//
//   S = Q K^T    Q [128 tokens x D] and K [128 keys x D] from shared memory, S in tensor memory
//                (one lane per token, one column per key), double-buffered
//   O += P V     P (bfloat16) read from tensor memory, where the softmax wrote it over S;
//                V [128 keys x D] from shared memory as the MN-major operand
//
//   warps 0-3  softmax: thread r owns token r.  It reads its row of S (tcgen05.ld), masks it on
//              tiles that touch the diagonal, the window's edge or the sequence's end, and writes
//              P = 2^(s*c - m*c) back as bfloat16 (tcgen05.st).  The running maximum m is only
//              raised when a row maximum exceeds it by more than 8 in the exponent; then the
//              thread rescales its row of O in tensor memory.  The sum of P is kept in float32.
//              At the end the thread divides its row of O by the sum and stores it.
//   warp 4     TMA producer: Q once, then K and V tiles through rings of two stages.  Rows of a V
//              tile that the cache never wrote (after the sequence's last position, or in a page
//              the sequence does not hold) are cleared in shared memory, so that a weight of
//              zero cannot meet a stray NaN.
//   warp 5     allocates tensor memory; one lane issues the tcgen05.mma and commits them to the
//              barriers that the other warps wait on.
//
// Every wait on an mbarrier is bounded: a wait that runs out records BFI_STATUS_TIMEOUT in the
// status word, every role leaves its loop, outstanding copies get a bounded time to land, and the
// block frees its tensor memory and returns.
#include "tcgen05.cuh"

#define FT_THREADS 192
#define FT_ROWS 128           // tokens per block
#define FT_KEYS 128           // keys per tile: two pages
#define FT_PAGE 64
#define FT_BOX_BYTES (128 * 128)      // a box of 128 rows x 64 bfloat16
#define FT_RESCALE_ABOVE 8.0f         // in the exponent of 2: P stays below 2^8

// 32 consecutive columns of this thread's lane; the caller waits with tmem_wait_ld()
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
          "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]),
          "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]),
          "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (bfloat16, two values per 32-bit column) comes from tensor memory
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc)
        : "memory");
}
// Shared-memory descriptor of an MN-major operand with the 128-byte swizzle: 64 consecutive values
// of the M/N side are one 128-byte row, 8 rows (8 steps of k) one 1024-byte group.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor with B taken MN-major (bit 16)
__host__ __device__ constexpr uint32_t umma_idesc_b_mn(int m, int n) { return umma_idesc(m, n) | (1u << 16); }

__device__ __forceinline__ float ft_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t ft_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(FT_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, long out_stride,
                            const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int n_q, int n_kv,
                            int window, float scale_log2, uint32_t v_lbo, uint32_t v_sbo, int* __restrict__ status) {
    constexpr int BOXES = D / 64;
    constexpr int TILE_BYTES = BOXES * FT_BOX_BYTES;       // the Q tile, a K tile or a V tile
    constexpr int PAGE_BYTES = FT_PAGE * 128;              // one page's rows inside a box
    constexpr int S_COLS = FT_KEYS;                        // columns of one S buffer
    constexpr int O_COL = 2 * S_COLS;                      // O behind the two S buffers

    // Blocks are handed to the SMs in the order x, y, z: the token tile is z, counted from the end,
    // so that every head's and sequence's longest tiles run first and the short ones fill the tail.
    const int seq = blockIdx.y;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int t0 = cu_seqlens[seq];
    const int nt = cu_seqlens[seq + 1] - t0;
    const int tok0 = ((int)gridDim.z - 1 - (int)blockIdx.z) * FT_ROWS;
    if (tok0 >= nt) return;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_smem = smem;
    unsigned char* k_smem = q_smem + TILE_BYTES;            // [2] stages
    unsigned char* v_smem = k_smem + 2 * TILE_BYTES;        // [2] stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + 2 * TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;      // [2]
    uint64_t* k_empty = bars + 3;     // [2]
    uint64_t* v_full = bars + 5;      // [2]
    uint64_t* v_empty = bars + 7;     // [2]
    uint64_t* s_full = bars + 9;      // [2]
    uint64_t* p_full = bars + 11;     // [2]
    uint64_t* o_ready = bars + 13;
    uint64_t* tail_bar = bars + 14;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* s_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int start = seq_start[seq];
    const int head = blockIdx.x;
    const int kvh = head / (n_q / n_kv);
    const int seq_hi = start + nt - 1;                                  // last position the cache holds
    const int p0 = start + tok0;                                        // position of the block's first token
    const int hi_block = start + min(tok0 + FT_ROWS - 1, nt - 1);
    const int lo_block = window > 0 ? max(0, p0 - window + 1) : 0;
    const int j_beg = lo_block / FT_KEYS, j_end = hi_block / FT_KEYS;   // key tiles, inclusive
    const int n_tiles = j_end - j_beg + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], FT_ROWS);
        }
        mbar_init(o_ready, 1);
        mbar_init(tail_bar, 1);
        *s_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();
    pdl_wait();

    if (warp == 4) {
        // ---------------------------------------------------------------- TMA producer
        const int* table = block_table + (size_t)slot * table_stride;
        if (lane == 0) {
            mbar_expect_tx(q_full, TILE_BYTES);
            for (int c = 0; c < BOXES; ++c) tma_load_2d(q_smem + c * FT_BOX_BYTES, &map_q, head * D + c * 64, t0 + tok0, q_full);
        }
        uint32_t tail_phase = 0;
        bool failed = false;
        for (int i = 0; i < n_tiles; ++i) {
            const int j = j_beg + i, st = i & 1;
            const uint32_t ph = (i >> 1) & 1;
            int pg[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int idx = 2 * j + h;
                pg[h] = idx < table_stride ? table[idx] : -1;
            }
            const int n_have = (pg[0] >= 0) + (pg[1] >= 0);
            unsigned char* kt = k_smem + (size_t)st * TILE_BYTES;
            unsigned char* vt = v_smem + (size_t)st * TILE_BYTES;
            int ok = 1;
            if (lane == 0) {
                if (i >= 2 && !mbar_wait(&k_empty[st], ph ^ 1)) ok = 0;
                if (ok) {
                    mbar_expect_tx(&k_full[st], n_have * BOXES * PAGE_BYTES);
                    for (int h = 0; h < 2; ++h)
                        if (pg[h] >= 0)
                            for (int c = 0; c < BOXES; ++c)
                                tma_load_2d(kt + c * FT_BOX_BYTES + h * PAGE_BYTES, &map_k, c * 64, (pg[h] * n_kv + kvh) * FT_PAGE,
                                            &k_full[st]);
                    if (i >= 2 && !mbar_wait(&v_empty[st], ph ^ 1)) ok = 0;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { failed = true; break; }
            if (__shfl_sync(0xffffffffu, *s_flag, 0)) break;
            const bool fix = n_have < 2 || j * FT_KEYS + FT_KEYS - 1 > seq_hi;
            if (!fix) {
                if (lane == 0) {
                    mbar_expect_tx(&v_full[st], 2 * BOXES * PAGE_BYTES);
                    for (int h = 0; h < 2; ++h)
                        for (int c = 0; c < BOXES; ++c)
                            tma_load_2d(vt + c * FT_BOX_BYTES + h * PAGE_BYTES, &map_v, c * 64, (pg[h] * n_kv + kvh) * FT_PAGE,
                                        &v_full[st]);
                }
            } else {
                // the tile has rows the cache never wrote: land it first, clear those rows, then hand it over
                if (lane == 0 && n_have > 0) {
                    mbar_expect_tx(tail_bar, n_have * BOXES * PAGE_BYTES);
                    for (int h = 0; h < 2; ++h)
                        if (pg[h] >= 0)
                            for (int c = 0; c < BOXES; ++c)
                                tma_load_2d(vt + c * FT_BOX_BYTES + h * PAGE_BYTES, &map_v, c * 64,
                                            (pg[h] * n_kv + kvh) * FT_PAGE, tail_bar);
                    if (!mbar_wait(tail_bar, tail_phase)) ok = 0;
                }
                if (n_have > 0) tail_phase ^= 1;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { failed = true; break; }
                for (int idx = lane; idx < FT_KEYS * 8 * BOXES; idx += 32) {
                    const int row = idx / (8 * BOXES), rest = idx - row * (8 * BOXES);
                    const int c = rest >> 3, chunk = rest & 7;
                    const bool stale = pg[row / FT_PAGE] < 0 || j * FT_KEYS + row > seq_hi;
                    if (stale) *reinterpret_cast<uint4*>(vt + c * FT_BOX_BYTES + row * 128 + chunk * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&v_full[st]);
            }
        }
        if (failed && lane == 0) {
            atomicOr(status, BFI_STATUS_TIMEOUT);
            *s_flag = 1;
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------------- tensor-core issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(FT_ROWS, FT_KEYS);
            constexpr uint32_t idesc_o = umma_idesc_b_mn(FT_ROWS, D);
            const uint32_t q_addr = smem_u32(q_smem);
            auto issue_qk = [&](int i) {          // S[i & 1] = Q K(i)^T
                const uint32_t k_addr = smem_u32(k_smem + (size_t)(i & 1) * TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (uint32_t)(kk >> 2) * FT_BOX_BYTES + (uint32_t)(kk & 3) * 32;
                    umma_bf16(tmem_base + (uint32_t)(i & 1) * S_COLS, umma_desc_sw128(q_addr + off), umma_desc_sw128(k_addr + off),
                              idesc_s, kk > 0);
                }
            };
            bool ok = mbar_wait(q_full, 0) && mbar_wait(&k_full[0], 0);
            if (ok) {
                tc_fence_after();
                issue_qk(0);
                umma_commit(&s_full[0]);
                umma_commit(&k_empty[0]);
            }
            for (int i = 0; ok && i < n_tiles && !*s_flag; ++i) {
                const int b = i & 1;
                const uint32_t ph = (i >> 1) & 1;
                if (i + 1 < n_tiles) {
                    if (!mbar_wait(&k_full[b ^ 1], ((i + 1) >> 1) & 1)) { ok = false; break; }
                    tc_fence_after();
                    issue_qk(i + 1);
                    umma_commit(&s_full[b ^ 1]);
                    umma_commit(&k_empty[b ^ 1]);
                }
                if (!mbar_wait(&p_full[b], ph) || !mbar_wait(&v_full[b], ph)) { ok = false; break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(v_smem + (size_t)b * TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < FT_KEYS / 16; ++kk)       // 16 keys per step: 8 columns of packed P, 2048 bytes of V
                    umma_bf16_a_tmem(tmem_base + O_COL, tmem_base + (uint32_t)b * S_COLS + kk * 8,
                                     umma_desc_mn_sw128(v_addr + kk * 2048, v_lbo, v_sbo), idesc_o, (i > 0 || kk > 0));
                umma_commit(&v_empty[b]);
                umma_commit(o_ready);
            }
            if (!ok) {
                atomicOr(status, BFI_STATUS_TIMEOUT);
                *s_flag = 1;
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax and output
        const int r = threadIdx.x;                                       // token of this thread, TMEM lane
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
        const int pos_r = min(p0 + r, seq_hi);
        const int lo_r = window > 0 ? max(0, pos_r - window + 1) : 0;
        float m_used = -INFINITY, l_run = 0.0f;
        bool ok = true, timed_out = false;
        // every wait's outcome is agreed on by the whole warp: the tensor-memory accesses are warp-wide
        for (int i = 0; i < n_tiles; ++i) {
            if (__any_sync(0xffffffffu, *s_flag != 0)) { ok = false; break; }
            const int j = j_beg + i, b = i & 1;
            const uint32_t ph = (i >> 1) & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(&s_full[b], ph))) { ok = false; timed_out = true; break; }
            tc_fence_after();
            float s[FT_KEYS];
            const uint32_t s_addr = lane_base + (uint32_t)b * S_COLS;
#pragma unroll
            for (int c = 0; c < FT_KEYS / 32; ++c) tmem_ld32(s_addr + c * 32, s + c * 32);
            tmem_wait_ld();
            const int key0 = j * FT_KEYS;
            const bool masked = key0 + FT_KEYS - 1 > p0 || key0 + FT_KEYS - 1 > seq_hi ||
                                (window > 0 && key0 < p0 + FT_ROWS - 1 - window + 1);
            if (masked) {
                const int hi = pos_r - key0, lo = lo_r - key0;       // keep lo <= index <= hi
#pragma unroll
                for (int e = 0; e < FT_KEYS; ++e)
                    if (e > hi || e < lo) s[e] = -INFINITY;
            }
            float mx = s[0];
#pragma unroll
            for (int e = 1; e < FT_KEYS; ++e) mx = fmaxf(mx, s[e]);
            // raise the running maximum only when a score would otherwise exceed 2^8 after the shift
            const bool raise = mx > -INFINITY && (m_used == -INFINITY || (mx - m_used) * scale_log2 > FT_RESCALE_ABOVE);
            if (__any_sync(0xffffffffu, raise && i > 0)) {
                const float m_new = raise ? mx : m_used;
                const float f = (raise && m_used > -INFINITY) ? ft_exp2((m_used - m_new) * scale_log2) : 1.0f;
                if (!__all_sync(0xffffffffu, mbar_wait(o_ready, (uint32_t)((i - 1) & 1)))) {     // O holds tiles 0 .. i-1
                    ok = false;
                    timed_out = true;
                    break;
                }
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    float o[32];
                    uint32_t ou[32];
                    tmem_ld32(lane_base + O_COL + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; ++e) ou[e] = __float_as_uint(o[e] * f);
                    tmem_st32(lane_base + O_COL + c * 32, ou);
                }
                l_run *= f;
                m_used = m_new;
            } else if (raise) {
                m_used = mx;                                          // first tile: nothing accumulated yet
            }
            const float mc = m_used == -INFINITY ? 0.0f : m_used * scale_log2;
            float sum = 0.0f;
            uint32_t pk[FT_KEYS / 2];
#pragma unroll
            for (int e = 0; e < FT_KEYS; e += 2) {
                const float a = ft_exp2(fmaf(s[e], scale_log2, -mc));
                const float c2 = ft_exp2(fmaf(s[e + 1], scale_log2, -mc));
                sum += a + c2;
                pk[e >> 1] = ft_pack(a, c2);
            }
            l_run += sum;
#pragma unroll
            for (int c = 0; c < FT_KEYS / 64; ++c) tmem_st32(s_addr + c * 32, pk + c * 32);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&p_full[b]);
        }
        if (ok && !__all_sync(0xffffffffu, mbar_wait(o_ready, (uint32_t)((n_tiles - 1) & 1)))) {
            ok = false;
            timed_out = true;
        }
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            const bool store = tok0 + r < nt;
            bf16* dst = out + (size_t)(t0 + tok0 + r) * out_stride + (size_t)head * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                float o[32];
                tmem_ld32(lane_base + O_COL + c * 32, o);
                tmem_wait_ld();
                if (store) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 w;
                        w.x = ft_pack(o[e] * inv, o[e + 1] * inv);
                        w.y = ft_pack(o[e + 2] * inv, o[e + 3] * inv);
                        w.z = ft_pack(o[e + 4] * inv, o[e + 5] * inv);
                        w.w = ft_pack(o[e + 6] * inv, o[e + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + e) = w;
                    }
                }
            }
        }
        if (timed_out && lane == 0) {
            atomicOr(status, BFI_STATUS_TIMEOUT);
            *s_flag = 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*s_flag && warp == 4 && lane == 0) {
        // a wait ran out: give outstanding TMA writes a bounded time to land
        mbar_wait(q_full, 0);
        for (int s = 0; s < 2; ++s) {
            mbar_wait(&k_full[s], 0), mbar_wait(&k_full[s], 1);
            mbar_wait(&v_full[s], 0), mbar_wait(&v_full[s], 1);
        }
        mbar_wait(tail_bar, 0), mbar_wait(tail_bar, 1);
    }
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int D>
static int launch_prefill_tc(const void* qkv, long q_stride, void* out, long out_stride, const void* k_pages,
                             const void* v_pages, long n_pages, const int* block_table, int table_stride,
                             const int* cu_seqlens, const int* seq_slot, const int* seq_start, int n_seqs, long n_tokens,
                             int max_seq_tokens, int n_q, int n_kv, int window, float scale, int* status,
                             cudaStream_t stream) {
    CUtensorMap mq, mk, mv;
    int rc = bfi_tensor_map_bf16(qkv, n_tokens, (long)n_q * D, q_stride, FT_ROWS, &mq);
    if (rc) return rc;
    rc = bfi_tensor_map_bf16(k_pages, n_pages * n_kv * FT_PAGE, D, D, FT_PAGE, &mk);
    if (rc) return rc;
    rc = bfi_tensor_map_bf16(v_pages, n_pages * n_kv * FT_PAGE, D, D, FT_PAGE, &mv);
    if (rc) return rc;
    constexpr int TILE_BYTES = (D / 64) * FT_BOX_BYTES;
    // at least half an SM's shared memory, so that two blocks never share one SM's tensor memory
    const size_t tiles = (size_t)5 * TILE_BYTES + 1024 + 256;
    const size_t smem = tiles > 120 * 1024 ? tiles : 120 * 1024;
    auto kernel = attention_prefill_tc_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return bfi_fail("attention_prefill_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem,
                                          cudaGetErrorString(e));
    const unsigned lbo = FT_BOX_BYTES;      // leading byte offset: between the two 64-wide halves of the head
    const unsigned sbo = 1024;              // stride byte offset: between groups of 8 keys
    dim3 grid(n_q, n_seqs, (max_seq_tokens + FT_ROWS - 1) / FT_ROWS);
    bfi_launch(kernel, grid, dim3(FT_THREADS), smem, stream, mq, mk, mv, (bf16*)out, out_stride, block_table, table_stride,
               cu_seqlens, seq_slot, seq_start, n_q, n_kv, window, scale * 1.4426950408889634f, (uint32_t)lbo, (uint32_t)sbo,
               status);
    return bfi_check_launch("attention_prefill_tcgen05");
}

// qkv [n_tokens, >= n_q*d] with the step's query heads (already normalised and rotated), the
// cache pages [n_pages, n_kv, 64, d] holding every key and value up to each sequence's last new
// token.  Returns 0 on success, 1 on error, 2 when the shape is not taken (nothing launched):
// head sizes other than 64/128, or operands TMA cannot address.  A wait that ran out sets
// BFI_STATUS_TIMEOUT in `status`.
extern "C" int bfi_attention_prefill_tcgen05_bf16(const void* qkv, long q_stride, void* out, long out_stride,
                                                  const void* k_pages, const void* v_pages, long n_pages,
                                                  const int* block_table, int table_stride, const int* cu_seqlens,
                                                  const int* seq_slot, const int* seq_start, int n_seqs, long n_tokens,
                                                  int max_seq_tokens, int n_q, int n_kv, int d, int window, float scale,
                                                  int* status, cudaStream_t stream) {
    BFI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_prefill_tcgen05: %d query heads do not divide into %d kv heads",
                n_q, n_kv);
    BFI_REQUIRE(window >= 0 && status != nullptr, "attention_prefill_tcgen05: bad window or no status word");
    if (n_seqs <= 0 || max_seq_tokens <= 0) return 0;
    if (d != 64 && d != 128) return 2;
    if (q_stride % 8 != 0 || out_stride % 8 != 0 || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15) ||
        ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || n_seqs > 65535 ||
        (max_seq_tokens + FT_ROWS - 1) / FT_ROWS > 65535)
        return 2;
    if (n_pages * n_kv * FT_PAGE > 0x7fffffffL) return 2;       // TMA coordinates are 32-bit
    if (d == 64)
        return launch_prefill_tc<64>(qkv, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                     cu_seqlens, seq_slot, seq_start, n_seqs, n_tokens, max_seq_tokens, n_q, n_kv, window,
                                     scale, status, stream);
    return launch_prefill_tc<128>(qkv, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                  cu_seqlens, seq_slot, seq_start, n_seqs, n_tokens, max_seq_tokens, n_q, n_kv, window, scale,
                                  status, stream);
}
