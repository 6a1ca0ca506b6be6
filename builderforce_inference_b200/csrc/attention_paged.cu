// Causal grouped-query attention over the paged cache, for any step: whole prompts, prompts that
// continue a cached prefix, and single decoded tokens.  Float32 arithmetic with an online
// (max-subtracted) softmax; storage float32 or bfloat16.  This is the attention of the 32-bit
// path and the general fallback of the bfloat16 path.
//
// Reference formula (crates/bfi-core/src/cpu.rs:328-392): score = q.k / sqrt(d) for keys at or
// before the query's position, softmax over them, weighted sum of V; query head h reads kv head
// h / (n_q / n_kv).  `window` > 0 keeps only the last `window` keys (pos - window < j <= pos).
//
// Work split: one block per (sequence, kv head, chunk of heads of its group, chunk of tokens);
// 16 query rows per block (GH heads x 16/GH consecutive tokens) share each tile of 32 keys that
// is staged in shared memory as float32.  Within a warp a lane owns one key of the tile for the
// scores and a slice of head_dim for the output.
#include "common.cuh"

#define ATT_ROWS 16
#define ATT_KEYS 32
#define ATT_WARPS 8
#define ATT_MAX_D 512
#define ATT_MAX_NC (ATT_MAX_D / 32)

template <typename T, int NC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_paged_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                       const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                       const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int n_q, int n_kv, int d,
                       int gh, int head_chunks, int window, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* qs = smem;                          // [ATT_ROWS][d]
    float* ks = qs + ATT_ROWS * d;             // [ATT_KEYS][d + 1]
    float* vs = ks + ATT_KEYS * (d + 1);       // [ATT_KEYS][d]

    const int seq = blockIdx.z;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int t0 = cu_seqlens[seq];
    const int nt = cu_seqlens[seq + 1] - t0;
    const int qt = ATT_ROWS / gh;              // tokens per block
    const int tok0 = blockIdx.x * qt;
    if (tok0 >= nt) return;
    const int start = seq_start[seq];
    const int group = n_q / n_kv;
    const int kvh = blockIdx.y / head_chunks;
    const int hc = blockIdx.y - kvh * head_chunks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- stage the 16 query rows, scaled
    for (int i = threadIdx.x; i < ATT_ROWS * d; i += blockDim.x) {
        const int r = i / d, e = i - r * d;
        const int tok = tok0 + r / gh;
        const int hl = hc * gh + r % gh;
        float v = 0.0f;
        if (tok < nt && hl < group)
            v = to_f32(q[(size_t)(t0 + tok) * q_stride + (size_t)(kvh * group + hl) * d + e]) * scale;
        qs[i] = v;
    }

    // ---- the two rows of this warp
    int row_pos[2];
    bool row_ok[2];
    int row_lo[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = warp * 2 + i;
        const int tok = tok0 + r / gh;
        const int hl = hc * gh + r % gh;
        row_ok[i] = tok < nt && hl < group;
        row_pos[i] = start + tok;
        row_lo[i] = window > 0 ? max(0, row_pos[i] - window + 1) : 0;
    }
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.0f, 0.0f};
    float acc[2][NC];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[i][c] = 0.0f;

    // ---- key range of the block
    const int last_tok = min(tok0 + qt, nt) - 1;
    const int hi = start + last_tok;                                     // last key any row reads
    const int lo = window > 0 ? max(0, start + tok0 - window + 1) : 0;   // first key any row reads
    const size_t page_elems = (size_t)n_kv * BFI_PAGE_TOKENS * d;

    for (int kb = (lo / ATT_KEYS) * ATT_KEYS; kb <= hi; kb += ATT_KEYS) {
        __syncthreads();
        const int page = block_table[(size_t)slot * table_stride + kb / BFI_PAGE_TOKENS];
        const size_t base = (size_t)(page < 0 ? 0 : page) * page_elems +
                            ((size_t)kvh * BFI_PAGE_TOKENS + (kb % BFI_PAGE_TOKENS)) * d;
        for (int i = threadIdx.x; i < ATT_KEYS * d; i += blockDim.x) {
            const int j = i / d, e = i - j * d;
            const int key = kb + j;
            float kv = 0.0f, vv = 0.0f;
            if (page >= 0 && key >= lo && key <= hi) {
                kv = to_f32(k_pages[base + (size_t)j * d + e]);
                vv = to_f32(v_pages[base + (size_t)j * d + e]);
            }
            ks[j * (d + 1) + e] = kv;
            vs[j * d + e] = vv;
        }
        __syncthreads();

        const int key = kb + lane;
        float s[2] = {0.0f, 0.0f};
        const float* kr = ks + lane * (d + 1);
        const float* q0 = qs + (warp * 2) * d;
        const float* q1 = q0 + d;
        for (int e = 0; e < d; ++e) {
            const float kk = kr[e];
            s[0] = fmaf(q0[e], kk, s[0]);
            s[1] = fmaf(q1[e], kk, s[1]);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const bool valid = row_ok[i] && page >= 0 && key <= row_pos[i] && key >= row_lo[i];
            const float sc = valid ? s[i] : -INFINITY;
            const float m_tile = warp_max(sc);
            if (m_tile == -INFINITY) continue;   // no key of this tile is visible to the row (uniform in the warp)
            const float m_new = fmaxf(m_run[i], m_tile);
            const float corr = expf(m_run[i] - m_new);          // exp(-inf) = 0 on the first tile
            const float p = valid ? expf(sc - m_new) : 0.0f;
            l_run[i] = l_run[i] * corr + warp_sum(p);
            m_run[i] = m_new;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[i][c] *= corr;
            for (int jj = 0; jj < ATT_KEYS; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                if (pj == 0.0f) continue;
                const float* vr = vs + jj * d;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int e = lane + 32 * c;
                    if (e < d) acc[i][c] = fmaf(pj, vr[e], acc[i][c]);
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!row_ok[i]) continue;
        const int r = warp * 2 + i;
        const int tok = tok0 + r / gh;
        const int hl = hc * gh + r % gh;
        const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
        T* o = out + (size_t)(t0 + tok) * out_stride + (size_t)(kvh * group + hl) * d;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int e = lane + 32 * c;
            if (e < d) o[e] = from_f32<T>(acc[i][c] * inv);
        }
    }
}

template <typename T, int NC>
static int launch_attention(const void* q, long q_stride, void* out, long out_stride, const void* k_pages,
                            const void* v_pages, const int* block_table, int table_stride, const int* cu_seqlens,
                            const int* seq_slot, const int* seq_start, int n_seqs, int max_tokens, int n_q, int n_kv,
                            int d, int window, float scale, cudaStream_t stream) {
    const int group = n_q / n_kv;
    int gh = 1;
    while (gh < group && gh < 8) gh *= 2;
    const int head_chunks = (group + gh - 1) / gh;
    const int qt = ATT_ROWS / gh;
    dim3 grid((max_tokens + qt - 1) / qt, n_kv * head_chunks, n_seqs);
    BFI_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "attention_paged: too many heads (%d) or sequences (%d) for one launch",
                (int)grid.y, n_seqs);
    const size_t smem = (size_t)(ATT_ROWS * d + ATT_KEYS * (d + 1) + ATT_KEYS * d) * sizeof(float);
    auto kernel = attention_paged_kernel<T, NC>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return bfi_fail("attention_paged: cannot reserve %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
    }
    bfi_launch(kernel, dim3(grid), dim3(ATT_WARPS * 32), smem, stream, (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pages,
                                                   (const T*)v_pages, block_table, table_stride, cu_seqlens, seq_slot,
                                                   seq_start, n_q, n_kv, d, gh, head_chunks, window, scale);
    return bfi_check_launch("attention_paged");
}

template <typename T>
static int dispatch_nc(int nc, const void* q, long q_stride, void* out, long out_stride, const void* k_pages,
                       const void* v_pages, const int* block_table, int table_stride, const int* cu_seqlens,
                       const int* seq_slot, const int* seq_start, int n_seqs, int max_tokens, int n_q, int n_kv, int d,
                       int window, float scale, cudaStream_t stream) {
#define BFI_ATT_CASE(N)                                                                                              \
    case N:                                                                                                          \
        return launch_attention<T, N>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,     \
                                      cu_seqlens, seq_slot, seq_start, n_seqs, max_tokens, n_q, n_kv, d, window,     \
                                      scale, stream);
    switch (nc) {
        BFI_ATT_CASE(1)
        BFI_ATT_CASE(2)
        BFI_ATT_CASE(3)
        BFI_ATT_CASE(4)
        BFI_ATT_CASE(6)
        BFI_ATT_CASE(8)
        BFI_ATT_CASE(16)
        default:
            break;
    }
#undef BFI_ATT_CASE
    return bfi_fail("attention_paged: no kernel for head_dim %d", d);
}

extern "C" int bfi_attention_paged(const void* q, int dtype, long q_stride, void* out, long out_stride,
                                   const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                                   const int* cu_seqlens, const int* seq_slot, const int* seq_start, int n_seqs,
                                   int max_tokens, int n_q, int n_kv, int d, int window, float scale,
                                   cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "attention_paged: unknown dtype code %d", dtype);
    BFI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_paged: %d query heads do not divide into %d kv heads",
                n_q, n_kv);
    BFI_REQUIRE(d > 0 && d % 16 == 0 && d <= ATT_MAX_D, "attention_paged: head_dim %d must be a multiple of 16, at most %d",
                d, ATT_MAX_D);
    BFI_REQUIRE(window >= 0, "attention_paged: negative window");
    BFI_REQUIRE(q_stride >= (long)n_q * d && out_stride >= (long)n_q * d, "attention_paged: token stride shorter than the heads");
    if (n_seqs <= 0 || max_tokens <= 0) return 0;
    // round the slice count up to an instantiated value
    int nc = (d + 31) / 32;
    if (nc == 5) nc = 6;
    if (nc == 7) nc = 8;
    if (nc > 8) nc = 16;
    if (dtype == BFI_F32)
        return dispatch_nc<float>(nc, q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                                  cu_seqlens, seq_slot, seq_start, n_seqs, max_tokens, n_q, n_kv, d, window, scale, stream);
    return dispatch_nc<bf16>(nc, q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride, cu_seqlens,
                             seq_slot, seq_start, n_seqs, max_tokens, n_q, n_kv, d, window, scale, stream);
}
