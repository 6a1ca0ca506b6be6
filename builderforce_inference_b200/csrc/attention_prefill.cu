// Prompt attention for bfloat16 on the tensor cores: every new token of a step attends causally
// over the cached keys and values of its sequence (the step's own tokens are already in the cache),
// whole prompts and continuations of a cached prefix alike, with an optional window
// (crates/bfi-core/src/cpu.rs:328-392).
//
// One block per (sequence, query head, 64 consecutive tokens); each of its four warps owns 16
// tokens.  Keys and values arrive page by page (64 rows) through a two-stage cp.async ring in
// XOR-swizzled shared memory; scores and the output are mma.sync.m16n8k16 tiles with float32
// accumulators, the softmax is the online (running max / running sum) form in float32 with
// ex2.approx on scores pre-multiplied by log2(e).  A warp skips pages that lie wholly after its
// last token or wholly before its window.
#include "attention_tiles.cuh"

#define AP_QROWS 64

template <int D>
__global__ void __launch_bounds__(AD_THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out, long out_stride,
                         const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                         const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_seqlens,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int n_q, int n_kv,
                         int window, float scale_log2) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);                       // [64][D]
    bf16* ks[2] = {qs + AP_QROWS * D, qs + AP_QROWS * D + 2 * AD_TILE * D};
    bf16* vs[2] = {ks[0] + AD_TILE * D, ks[1] + AD_TILE * D};

    const int seq = blockIdx.z;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int t0 = cu_seqlens[seq];
    const int nt = cu_seqlens[seq + 1] - t0;
    const int tok0 = blockIdx.x * AP_QROWS;
    if (tok0 >= nt) return;
    const int start = seq_start[seq];
    const int head = blockIdx.y;
    const int kvh = head / (n_q / n_kv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const int seq_hi = start + nt - 1;                                   // last key the cache holds for this sequence
    const int hi_block = start + min(tok0 + AP_QROWS - 1, nt - 1);       // last key any row of the block reads
    const int lo_block = window > 0 ? max(0, start + tok0 - window + 1) : 0;
    const int p_beg = lo_block / AD_TILE, p_end = hi_block / AD_TILE;    // inclusive

    // ---- Q tile -> shared memory (rows past the sequence are zero)
    {
        constexpr int CHUNKS = D / 8;
        for (int i = threadIdx.x; i < AP_QROWS * CHUNKS; i += AD_THREADS) {
            const int row = i / CHUNKS, c = i - row * CHUNKS;
            bf16* dst = qs + row * D + ((c ^ (row & 7)) << 3);
            if (tok0 + row < nt)
                cp_async16(dst, q + (size_t)(t0 + tok0 + row) * q_stride + (size_t)head * D + c * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    const size_t page_elems = (size_t)n_kv * AD_TILE * D;
    const int* table = block_table + (size_t)slot * table_stride;
    auto issue = [&](int page_idx, int stage) {
        const int page = table[page_idx];
        if (page >= 0) {
            const size_t base = (size_t)page * page_elems + (size_t)kvh * AD_TILE * D;
            load_tile<D>(ks[stage], k_pages + base);
            load_tile<D>(vs[stage], v_pages + base);
        }
        cp_async_commit();
    };
    issue(p_beg, 0);                     // the Q copies ride in this first group

    // rows of this warp: tokens tok0 + 16*warp + g and + 8
    int pos_r[2], lo_r[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        pos_r[r] = start + tok0 + warp * 16 + g + r * 8;
        lo_r[r] = window > 0 ? max(0, pos_r[r] - window + 1) : 0;
    }
    const int warp_pos_max = start + tok0 + warp * 16 + 15;
    const int warp_lo_min = window > 0 ? max(0, start + tok0 + warp * 16 - window + 1) : 0;

    uint32_t qa[D / 16][4];
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.0f, 0.0f};
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;

    for (int p = p_beg; p <= p_end; ++p) {
        const int stage = (p - p_beg) & 1;
        if (p + 1 <= p_end) {
            issue(p + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (p == p_beg) {
            // query fragments: 16 rows of this warp, all of D
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int row = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                ldmatrix_x4(qa[kk], tile_chunk<D>(qs, row, 2 * kk + (lane >> 4)));
            }
        }
        const bool have_page = table[p] >= 0;
        const bf16* kt = ks[stage];
        const bf16* vt = vs[stage];
        if ((p + 1) * AD_TILE - 1 > seq_hi) {
            // the sequence's last page: rows after its last token were never written; a zero weight
            // times a stray NaN would still poison the output, so clear those value rows
            const int first_bad = seq_hi - p * AD_TILE + 1;
            constexpr int CHUNKS = D / 8;
            for (int i = threadIdx.x; i < (AD_TILE - first_bad) * CHUNKS; i += AD_THREADS) {
                const int row = first_bad + i / CHUNKS, c = i % CHUNKS;
                *reinterpret_cast<uint4*>(vs[stage] + row * D + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncthreads();
        }
        const int key_lo = p * AD_TILE, key_hi = key_lo + AD_TILE - 1;
        if (have_page && key_lo <= warp_pos_max && key_hi >= warp_lo_min) {
            // ---- scores: 16 tokens x 64 keys
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[j][i] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < D / 16; kk += 2) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint32_t b[4];
                    ldmatrix_x4(b, tile_chunk<D>(kt, j * 8 + (lane & 7), 2 * kk + (lane >> 3)));
                    mma16816(s[j], qa[kk], b[0], b[1]);
                    mma16816(s[j], qa[kk + 1], b[2], b[3]);
                }
            }
            // ---- mask (only where the page crosses a row's limits) and online softmax
            const bool need_mask = key_hi > start + tok0 + warp * 16 || key_lo < (window > 0 ? warp_pos_max - window + 1 : 0);
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        float v = s[j][r * 2 + c] * scale_log2;
                        if (need_mask) {
                            const int key = key_lo + j * 8 + 2 * t + c;
                            if (key > pos_r[r] || key < lo_r[r]) v = -INFINITY;
                        }
                        s[j][r * 2 + c] = v;
                        mx = fmaxf(mx, v);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[r], mx);
                const float corr = (m_run[r] == -INFINITY) ? 0.0f : fast_exp2(m_run[r] - m_new);
                float sum = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const float v = s[j][r * 2 + c];
                        const float pv = (v == -INFINITY) ? 0.0f : fast_exp2(v - m_new);
                        s[j][r * 2 + c] = pv;
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
            // ---- output += P V, 16 keys at a time
#pragma unroll
            for (int ks4 = 0; ks4 < 4; ++ks4) {
                uint32_t pa[4];
                pa[0] = pack_bf16(s[2 * ks4][0], s[2 * ks4][1]);
                pa[1] = pack_bf16(s[2 * ks4][2], s[2 * ks4][3]);
                pa[2] = pack_bf16(s[2 * ks4 + 1][0], s[2 * ks4 + 1][1]);
                pa[3] = pack_bf16(s[2 * ks4 + 1][2], s[2 * ks4 + 1][3]);
#pragma unroll
                for (int dd = 0; dd < D / 8; dd += 2) {
                    uint32_t b[4];
                    const int row = ks4 * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    ldmatrix_x4_trans(b, tile_chunk<D>(vt, row, dd + (lane >> 4)));
                    mma16816(o[dd], pa, b[0], b[1]);
                    mma16816(o[dd + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();          // the stage is free for the load issued in the next iteration
    }

    // ---- normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int tok = tok0 + warp * 16 + g + r * 8;
        if (tok >= nt) continue;
        const float inv = l_run[r] > 0.0f ? 1.0f / l_run[r] : 0.0f;
        bf16* orow = out + (size_t)(t0 + tok) * out_stride + (size_t)head * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const __nv_bfloat162 v2 = __floats2bfloat162_rn(o[i][r * 2] * inv, o[i][r * 2 + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(orow + i * 8 + 2 * t) = v2;
        }
    }
}

template <int D>
static int launch_prefill(const void* q, long q_stride, void* out, long out_stride, const void* k_pages,
                          const void* v_pages, const int* block_table, int table_stride, const int* cu_seqlens,
                          const int* seq_slot, const int* seq_start, int n_seqs, int max_tokens, int n_q, int n_kv,
                          int window, float scale, cudaStream_t stream) {
    const size_t smem = (size_t)(AP_QROWS * D + 4 * AD_TILE * D) * sizeof(bf16);
    auto kernel = attention_prefill_kernel<D>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return bfi_fail("attention_prefill: cannot reserve %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
    }
    dim3 grid((max_tokens + AP_QROWS - 1) / AP_QROWS, n_q, n_seqs);
    bfi_launch(kernel, grid, dim3(AD_THREADS), smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride,
               (const bf16*)k_pages, (const bf16*)v_pages, block_table, table_stride, cu_seqlens, seq_slot, seq_start, n_q,
               n_kv, window, scale * 1.4426950408889634f);
    return bfi_check_launch("attention_prefill");
}

// Returns 0 on success, 1 on error, 2 when the shape is not taken (nothing launched).
extern "C" int bfi_attention_prefill_bf16(const void* q, long q_stride, void* out, long out_stride, const void* k_pages,
                                          const void* v_pages, const int* block_table, int table_stride,
                                          const int* cu_seqlens, const int* seq_slot, const int* seq_start, int n_seqs,
                                          int max_tokens, int n_q, int n_kv, int d, int window, float scale,
                                          cudaStream_t stream) {
    BFI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_prefill: %d query heads do not divide into %d kv heads",
                n_q, n_kv);
    BFI_REQUIRE(window >= 0, "attention_prefill: negative window");
    if (n_seqs <= 0 || max_tokens <= 0) return 0;
    if (d != 64 && d != 128) return 2;
    if (q_stride % 8 != 0 || out_stride % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)out & 3) || n_seqs > 65535 ||
        n_q > 65535)
        return 2;
    if (d == 64)
        return launch_prefill<64>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride, cu_seqlens,
                                  seq_slot, seq_start, n_seqs, max_tokens, n_q, n_kv, window, scale, stream);
    return launch_prefill<128>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride, cu_seqlens,
                               seq_slot, seq_start, n_seqs, max_tokens, n_q, n_kv, window, scale, stream);
}
