// Decode attention for bfloat16: one new token per sequence attends over its cached keys and
// values (crates/bfi-core/src/cpu.rs:328-392 with T = 1).  The step is bound by reading the cache
// once, so the work is split over (sequence, kv head, range of pages): each block streams its
// pages of 64 keys through a two-stage ring in shared memory -- one thread asks TMA for a page's
// keys and values (boxes of 64 rows x 128 bytes, 128-byte swizzle: the layout ldmatrix reads
// without bank conflicts), an mbarrier per stage says when they have landed -- all query heads of
// the group share the loaded keys and values (they are the 16 rows of the tensor-core tiles), and
// partial results (running maximum, sum and unnormalised output, float32) go to a scratch buffer.
// They are merged in range order by a second kernel (which, launched as a programmatic dependent,
// is already resident when the first one ends).
//
// Scores, the running maximum and sum, and the output accumulator are float32; exp is
// ex2.approx on scores pre-multiplied by log2(e).
//
// Every wait on an mbarrier is bounded: a wait that runs out records BFI_STATUS_TIMEOUT in the
// status word, the block gives its outstanding copies a bounded time to land and returns.
#include "attention_tiles.cuh"
#include "tcgen05.cuh"

// A sequence's pages are cut into at most `max_splits` ranges of equal size (in pages), so every
// sequence, long or short, spreads over the same number of blocks.
__device__ __forceinline__ int decode_pages_per_split(int n_pages, int max_splits) {
    return (n_pages + max_splits - 1) / max_splits;
}

// A tile as TMA leaves it: D/64 boxes of [64 rows][64 values] one after the other, the 16-byte
// chunk c of a box's row r at chunk c ^ (r & 7).  The tile starts on a 1024-byte boundary.
template <int D>
__device__ __forceinline__ bf16* box_chunk(bf16* tile, int row, int chunk) {
    return tile + (chunk >> 3) * (AD_TILE * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

#define AD_MERGE_PAD 8

template <int D>
struct DecodeSmem {
    static constexpr int TILE_BYTES = AD_TILE * D * 2;            // keys or values of one page and kv head
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int RING_BYTES = 2 * STAGE_BYTES;
    static constexpr int MERGE_BYTES = AD_WARPS * 16 * (2 + D + AD_MERGE_PAD) * 4;
    static constexpr int BODY_BYTES = RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES;
    static constexpr size_t BYTES = (size_t)BODY_BYTES + 64 /*barriers*/ + 1024 /*alignment*/;
};

// part_o  [seqs, n_q, max_splits, D]  float32 unnormalised outputs
// part_ml [seqs, n_q, max_splits, 2]  float32 (running max in log2 units, running sum)
template <int D>
__global__ void __launch_bounds__(AD_THREADS)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out, long out_stride,
                        const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_start, int n_q, int n_kv, int window, float scale_log2,
                        int head_chunks, float* __restrict__ part_o, float* __restrict__ part_ml,
                        int* __restrict__ status, TcWaits waits) {
    pdl_trigger();
    const uint32_t spin_limit = waits.spin_limit;
    using Smem = DecodeSmem<D>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + Smem::BODY_BYTES);       // [2]

    const int seq = blockIdx.z;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int max_splits = gridDim.x, split = blockIdx.x;
    const int group = n_q / n_kv;
    const int kvh = blockIdx.y / head_chunks;
    const int hc = blockIdx.y - kvh * head_chunks;
    const int head0 = kvh * group + hc * 16;              // first query head of this block
    const int n_heads = min(16, group - hc * 16);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const int pos = seq_start[seq];                       // the new token's position; keys lo..pos
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int first_page = lo / AD_TILE, last_page = pos / AD_TILE;
    const int n_pages = last_page - first_page + 1;
    const int pages_per_split = decode_pages_per_split(n_pages, max_splits);
    const int n_splits = (n_pages + pages_per_split - 1) / pages_per_split;    // ranges this sequence has
    if (split >= n_splits) return;
    const int p_beg = first_page + split * pages_per_split;
    const int p_end = min(last_page + 1, p_beg + pages_per_split);
    const int n_tiles = p_end - p_beg;

    const int* table = block_table + (size_t)slot * table_stride;
    if (threadIdx.x == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // thread 0 only: the keys and values of page `page_idx` of the sequence into stage `stage`
    auto issue = [&](int page_idx, int stage) {
        const int page = table[page_idx];
        if (page >= 0) {
            bf16* kt = reinterpret_cast<bf16*>(smem + (size_t)stage * Smem::STAGE_BYTES);
            bf16* vt = kt + AD_TILE * D;
            const int row = (page * n_kv + kvh) * AD_TILE;
            mbar_expect_tx(&full[stage], Smem::STAGE_BYTES);
#pragma unroll
            for (int h = 0; h < D / 64; ++h) {
                tma_load_2d(kt + h * (AD_TILE * 64), &map_k, h * 64, row, &full[stage]);
                tma_load_2d(vt + h * (AD_TILE * 64), &map_v, h * 64, row, &full[stage]);
            }
        } else {
            mbar_arrive(&full[stage]);                    // a page the sequence does not hold: nothing to wait for
        }
    };

    // The sequence's older pages, its slot, position and page table were all written before this
    // step's kernels began; only the page of the new token (the last one) and q come from the
    // kernel before this one.  So the first two tiles, unless they are that page, travel before the wait.
    int issued = 0;                                       // tiles on their way (thread 0 keeps count)
    const bool producer = threadIdx.x == 0 && !waits.hold_producer;
    if (producer)
        while (issued < 2 && issued < n_tiles && p_beg + issued != last_page) {
            issue(p_beg + issued, issued);
            ++issued;
        }
    pdl_wait();
    if (producer && issued == 0 && n_tiles > 0) {
        issue(p_beg, 0);
        issued = 1;
    }

    // query fragments: rows g and g+8 are heads head0+g, head0+g+8
    const bf16* qbase = q + (size_t)seq * q_stride;       // one token per sequence: row index = seq
    uint32_t qa[D / 16][4];
    {
        const bool ok_lo = g < n_heads, ok_hi = g + 8 < n_heads;
        const bf16* q_lo = qbase + (size_t)(head0 + g) * D;
        const bf16* q_hi = qbase + (size_t)(head0 + g + 8) * D;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int c = kk * 16 + 2 * t;
            qa[kk][0] = ok_lo ? *reinterpret_cast<const uint32_t*>(q_lo + c) : 0u;
            qa[kk][1] = ok_hi ? *reinterpret_cast<const uint32_t*>(q_hi + c) : 0u;
            qa[kk][2] = ok_lo ? *reinterpret_cast<const uint32_t*>(q_lo + c + 8) : 0u;
            qa[kk][3] = ok_hi ? *reinterpret_cast<const uint32_t*>(q_hi + c + 8) : 0u;
        }
    }

    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.0f, 0.0f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;

    bool ok = true;
    for (int it = 0; it < n_tiles; ++it) {
        const int p = p_beg + it;
        const int stage = it & 1;
        // the other stage was read for the last time before the barrier that ended the iteration before
        if (producer && it + 1 < n_tiles && it + 1 >= issued) {
            issue(p + 1, stage ^ 1);
            ++issued;
        }
        ok = __syncthreads_and(mbar_wait(&full[stage], (uint32_t)((it >> 1) & 1), spin_limit));
        if (!ok) break;                                   // the same for every thread of the block
        const bool have_page = table[p] >= 0;
        bf16* kt = reinterpret_cast<bf16*>(smem + (size_t)stage * Smem::STAGE_BYTES);
        bf16* vt = kt + AD_TILE * D;
        if ((p + 1) * AD_TILE - 1 > pos) {
            // the page that holds `pos`: its later rows were never written.  Their scores are masked,
            // but a weight of zero times a stray NaN would still poison the output, so clear them.
            const int first_bad = pos - p * AD_TILE + 1;
            constexpr int CHUNKS = D / 8;
            for (int i2 = threadIdx.x; i2 < (AD_TILE - first_bad) * CHUNKS; i2 += AD_THREADS) {
                const int row = first_bad + i2 / CHUNKS, c = i2 % CHUNKS;
                *reinterpret_cast<uint4*>(box_chunk<D>(vt, row, c)) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncthreads();
        }

        // ---- scores of this warp's 16 keys: two n-tiles of 8 keys
        // two accumulators per n-tile (even and odd k steps), added at the end: the chain of
        // dependent tensor-core instructions is half as long
        float s[2][4], s_odd[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i2 = 0; i2 < 4; ++i2) s[j][i2] = s_odd[j][i2] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk += 2) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                // four 8x8 matrices: key rows of n-tile j, chunks 2kk .. 2kk+3 (two k16 steps)
                uint32_t b[4];
                const int row = warp * 16 + j * 8 + (lane & 7);
                ldmatrix_x4(b, box_chunk<D>(kt, row, 2 * kk + (lane >> 3)));
                mma16816(s[j], qa[kk], b[0], b[1]);
                mma16816(s_odd[j], qa[kk + 1], b[2], b[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i2 = 0; i2 < 4; ++i2) s[j][i2] += s_odd[j][i2];
        // ---- mask and online softmax; c0,c1 -> row g, keys 2t,2t+1; c2,c3 -> row g+8
        const int key0 = p * AD_TILE + warp * 16;
        float p_frag[2][4];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (r == 1 && n_heads <= 8) {                 // rows 8..15 are heads this block does not have
                p_frag[0][2] = p_frag[0][3] = p_frag[1][2] = p_frag[1][3] = 0.0f;
                continue;
            }
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int key = key0 + j * 8 + 2 * t + c;
                    float v = s[j][r * 2 + c] * scale_log2;
                    if (!have_page || key > pos || key < lo) v = -INFINITY;
                    s[j][r * 2 + c] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[r], mx);
            const float corr = (m_run[r] == -INFINITY) ? 0.0f : fast_exp2(m_run[r] - m_new);
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const float v = s[j][r * 2 + c];
                    const float pv = (v == -INFINITY) ? 0.0f : fast_exp2(v - m_new);
                    p_frag[j][r * 2 + c] = pv;
                    sum += pv;
                }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_run[r] = l_run[r] * corr + sum;
            m_run[r] = m_new;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                o[i][r * 2] *= corr;
                o[i][r * 2 + 1] *= corr;
            }
        }
        // ---- P (16 heads x 16 keys) as the A operand, V rows of these 16 keys as B
        uint32_t pa[4];
        pa[0] = pack_bf16(p_frag[0][0], p_frag[0][1]);
        pa[1] = pack_bf16(p_frag[0][2], p_frag[0][3]);
        pa[2] = pack_bf16(p_frag[1][0], p_frag[1][1]);
        pa[3] = pack_bf16(p_frag[1][2], p_frag[1][3]);
        if (have_page) {
#pragma unroll
            for (int dd = 0; dd < D / 8; dd += 2) {
                uint32_t b[4];
                const int row = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                ldmatrix_x4_trans(b, box_chunk<D>(vt, row, dd + (lane >> 4)));
                mma16816(o[dd], pa, b[0], b[1]);
                mma16816(o[dd + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();      // the stage is free for the load issued in the next iteration
    }

    if (!ok) {
        // a wait ran out: say so, give the copies that were asked for a bounded time to land in
        // this block's shared memory, and leave without a result
        if (threadIdx.x == 0) {
            atomicOr(status, BFI_STATUS_TIMEOUT);
            for (int j = 0; j < issued; ++j)
                if (j + 2 >= issued) mbar_wait(&full[j & 1], (uint32_t)((j >> 1) & 1), spin_limit);
        }
        __syncthreads();
        return;
    }

    // ---- merge the four warps (each saw a quarter of every tile) through shared memory: only the
    // rows of heads that exist, rows AD_MERGE_PAD floats apart so that the lanes' pairs fall into distinct banks
    constexpr int LD = D + AD_MERGE_PAD;
    float* mm = reinterpret_cast<float*>(smem);                     // [warps][16][2]
    float* oo = mm + AD_WARPS * 16 * 2;                             // [warps][16][LD]
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + r * 8;
        if (row < n_heads) {
            if (t == 0) {
                mm[(warp * 16 + row) * 2] = m_run[r];
                mm[(warp * 16 + row) * 2 + 1] = l_run[r];
            }
#pragma unroll
            for (int i = 0; i < D / 8; ++i)
                *reinterpret_cast<float2*>(oo + (size_t)(warp * 16 + row) * LD + i * 8 + 2 * t) = make_float2(o[i][r * 2], o[i][r * 2 + 1]);
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < n_heads * D; idx += AD_THREADS) {
        const int row = idx / D, e = idx - row * D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) m = fmaxf(m, mm[(w * 16 + row) * 2]);
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < AD_WARPS; ++w) {
            const float mw = mm[(w * 16 + row) * 2];
            const float f = (mw == -INFINITY) ? 0.0f : fast_exp2(mw - m);
            l += mm[(w * 16 + row) * 2 + 1] * f;
            acc += oo[(size_t)(w * 16 + row) * LD + e] * f;
        }
        const int head = head0 + row;
        if (n_splits == 1) {
            out[(size_t)seq * out_stride + (size_t)head * D + e] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
        } else {
            const size_t pi = ((size_t)seq * n_q + head) * max_splits + split;
            part_o[pi * D + e] = acc;
            if (e == 0) {
                part_ml[pi * 2] = m;
                part_ml[pi * 2 + 1] = l;
            }
        }
    }
    BFI_TRACE_END();
}

// Merges the ranges of every (sequence, head) in range order.  CAP: the most ranges a sequence
// can have here (8, 16 or 32): every load of a thread is issued before the first is used, so the
// kernel costs one trip to memory after its wait; the sequence's slot and position, which were
// there before the step began, are fetched ahead of the wait.
template <int D, int CAP>
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                                              bf16* __restrict__ out, long out_stride, int n_q, int max_splits, int window) {
    pdl_trigger();
    const int seq = blockIdx.y, head = blockIdx.x;
    const int slot = seq_slot[seq];
    const int pos = seq_start[seq];
    pdl_wait();
    if (slot < 0) return;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_pages = pos / AD_TILE - lo / AD_TILE + 1;
    const int pps = decode_pages_per_split(n_pages, max_splits);
    const int n_splits = (n_pages + pps - 1) / pps;
    if (n_splits == 1) return;                            // the first kernel wrote the output itself
    const size_t base = ((size_t)seq * n_q + head) * max_splits;
    float ms[CAP], ls[CAP], os[CAP];
    const int e = threadIdx.x;                            // blockDim.x == D
#pragma unroll
    for (int s = 0; s < CAP; ++s) {
        const bool have = s < n_splits;
        ms[s] = have ? part_ml[(base + s) * 2] : -INFINITY;
        ls[s] = have ? part_ml[(base + s) * 2 + 1] : 0.0f;
        os[s] = have ? part_o[(base + s) * D + e] : 0.0f;
    }
    float m = ms[0];
#pragma unroll
    for (int s = 1; s < CAP; ++s) m = fmaxf(m, ms[s]);
    float l = 0.0f, acc = 0.0f;
#pragma unroll
    for (int s = 0; s < CAP; ++s) {
        const float f = (ms[s] == -INFINITY) ? 0.0f : fast_exp2(ms[s] - m);
        l += ls[s] * f;
        acc = fmaf(os[s], f, acc);
    }
    out[(size_t)seq * out_stride + (size_t)head * D + e] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
}

template <int D>
static int launch_decode(const void* q, long q_stride, void* out, long out_stride, const void* k_pages,
                         const void* v_pages, long n_pages, const int* block_table, int table_stride,
                         const int* seq_slot, const int* seq_start, int n_seqs, int n_q, int n_kv, int window, float scale,
                         int max_splits, float* part_o, float* part_ml, int* status, cudaStream_t stream, TcWaits waits) {
    CUtensorMap mk, mv;
    int rc = bfi_tensor_map_bf16(k_pages, n_pages * n_kv * AD_TILE, D, D, AD_TILE, &mk);
    if (rc) return rc;
    rc = bfi_tensor_map_bf16(v_pages, n_pages * n_kv * AD_TILE, D, D, AD_TILE, &mv);
    if (rc) return rc;
    const int group = n_q / n_kv;
    const int head_chunks = (group + 15) / 16;
    const size_t need = DecodeSmem<D>::BYTES;
    auto kernel = attention_decode_kernel<D>;
    if (need > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
        if (e != cudaSuccess) return bfi_fail("attention_decode: cannot reserve %zu bytes of shared memory: %s", need,
                                              cudaGetErrorString(e));
    }
    dim3 grid(max_splits, n_kv * head_chunks, n_seqs);
    const float scale_log2 = scale * 1.4426950408889634f;
    bfi_launch(kernel, grid, dim3(AD_THREADS), need, stream, mk, mv, (const bf16*)q, q_stride, (bf16*)out, out_stride,
               block_table, table_stride, seq_slot, seq_start, n_q, n_kv, window, scale_log2, head_chunks, part_o, part_ml,
               status, waits);
    rc = bfi_check_launch("attention_decode");
    if (rc || max_splits == 1) return rc;
#define BFI_MERGE(CAP)                                                                                                   \
    bfi_launch(attention_decode_merge_kernel<D, CAP>, dim3(n_q, n_seqs), dim3(D), 0, stream, (const float*)part_o,        \
               (const float*)part_ml, seq_slot, seq_start, (bf16*)out, out_stride, n_q, max_splits, window)
    if (max_splits <= 8) BFI_MERGE(8);
    else if (max_splits <= 16) BFI_MERGE(16);
    else BFI_MERGE(32);
#undef BFI_MERGE
    return bfi_check_launch("attention_decode_merge");
}

// The cache pages are [n_pages, n_kv, 64, d], contiguous.  Returns 0 on success, 1 on error, 2 when the
// shape is not taken (nothing launched): head sizes other than 64/128, or operands TMA cannot address.
// Every sequence's pages are cut into at most `max_splits` (up to 32) ranges.  With max_splits > 1 the caller
// gives part_o [n_seqs*n_q*max_splits*d] and part_ml [n_seqs*n_q*max_splits*2] floats.  `status` points at
// an int, zero before the first call, that gets BFI_STATUS_TIMEOUT when a wait for a page ran out.
static int attention_decode_launch(const void* q, long q_stride, void* out, long out_stride, const void* k_pages,
                                   const void* v_pages, long n_pages, const int* block_table, int table_stride,
                                   const int* seq_slot, const int* seq_start, int n_seqs, int n_q, int n_kv, int d,
                                   int window, float scale, int max_splits, float* part_o, float* part_ml, int* status,
                                   cudaStream_t stream, TcWaits waits) {
    BFI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_decode: %d query heads do not divide into %d kv heads",
                n_q, n_kv);
    BFI_REQUIRE(window >= 0 && max_splits >= 1 && max_splits <= 32, "attention_decode: bad window or split count (1..32)");
    BFI_REQUIRE(status != nullptr && n_pages > 0, "attention_decode: no status word or no pages");
    if (n_seqs <= 0) return 0;
    if (d != 64 && d != 128) return 2;
    if (q_stride % 8 != 0 || ((uintptr_t)q & 15) || n_seqs > 65535) return 2;
    if (((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || n_pages * n_kv * AD_TILE > 0x7fffffffL) return 2;
    if (max_splits > 1) BFI_REQUIRE(part_o && part_ml, "attention_decode: split runs need the scratch buffers");
    if (d == 64)
        return launch_decode<64>(q, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                 seq_slot, seq_start, n_seqs, n_q, n_kv, window, scale, max_splits, part_o, part_ml, status,
                                 stream, waits);
    return launch_decode<128>(q, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride, seq_slot,
                              seq_start, n_seqs, n_q, n_kv, window, scale, max_splits, part_o, part_ml, status, stream,
                              waits);
}

extern "C" int bfi_attention_decode_bf16(const void* q, long q_stride, void* out, long out_stride, const void* k_pages,
                                         const void* v_pages, long n_pages, const int* block_table, int table_stride,
                                         const int* seq_slot, const int* seq_start, int n_seqs, int n_q, int n_kv,
                                         int d, int window, float scale, int max_splits, float* part_o, float* part_ml,
                                         int* status, cudaStream_t stream) {
    return attention_decode_launch(q, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                   seq_slot, seq_start, n_seqs, n_q, n_kv, d, window, scale, max_splits, part_o, part_ml,
                                   status, stream, tc_waits_default());
}

// The same launch with its bounded waits cut to `spin_limit` polls and, with hold_producer, a thread
// that asks for no page at all: every wait for a page then runs out by construction.  The launch
// records BFI_STATUS_TIMEOUT in the status word, writes no output and returns; nothing faults and
// nothing waits without a bound.  For the tests of that path only.
extern "C" int bfi_attention_decode_bf16_wait_probe(const void* q, long q_stride, void* out, long out_stride,
                                                    const void* k_pages, const void* v_pages, long n_pages,
                                                    const int* block_table, int table_stride, const int* seq_slot,
                                                    const int* seq_start, int n_seqs, int n_q, int n_kv, int d,
                                                    int window, float scale, int max_splits, float* part_o,
                                                    float* part_ml, int* status, unsigned spin_limit, int hold_producer,
                                                    cudaStream_t stream) {
    BFI_REQUIRE(spin_limit > 0 && spin_limit <= TC_SPIN_LIMIT, "attention_decode probe: spin limit out of range");
    return attention_decode_launch(q, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                   seq_slot, seq_start, n_seqs, n_q, n_kv, d, window, scale, max_splits, part_o, part_ml,
                                   status, stream, TcWaits{spin_limit, hold_producer ? 1 : 0});
}

BFI_TRACE_EXPORT(attention_decode)
