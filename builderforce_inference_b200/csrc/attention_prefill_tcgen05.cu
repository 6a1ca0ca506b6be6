// Prompt attention for bfloat16 on the fifth-generation tensor cores: every new token of a step
// attends causally over the cached keys and values of its sequence (the step's own tokens are
// already in the cache), with an optional window (crates/bfi-core/src/cpu.rs:328-392).
//
// A work item is (sequence, query head, 128 consecutive tokens).  One block per SM draws items
// from a shared ticket counter until none is left: the token tiles from the last one down (the
// longest first, the short ones fill the tail), and within a tile index sequences and heads.  The
// rings of keys and values, the two score buffers and the tensor cores run on from one item into
// the next, so that an item's start-up and its output hide behind its neighbours' products.  Keys
// and values arrive as tiles of 128 positions (two cache pages) by TMA with the 128-byte swizzle;
// both products run as tcgen05.mma with float32 accumulators in tensor memory:
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
//              One tile into the next item (O is double-buffered too) the thread divides its row
//              of the finished item's O by the sum and stores it.
//   warp 4     TMA producer: draws the items, writes each item's record for the other warps,
//              loads its Q tile (two buffers), then K and V tiles through rings of two stages.  Rows of a V
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
#define FT_META_SEQS 512              // sequences whose numbers a block keeps in shared memory

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

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// A warp of the softmax group writes its 32 rows of a finished item's O, divided by the rows'
// sums, to `dst` (the warp's first row).  Rows leave through the warp's staging tile in shared
// memory (32 rows x 128 bytes, 16-byte units XOR-swizzled by the row), so that a store instruction
// of the warp writes four whole 128-byte lines instead of 16 bytes of 32 different rows.
template <int D>
__device__ __noinline__ bool ft_write_out(uint64_t* o_done, uint32_t parity, uint64_t* o_free, uint32_t o_addr, float l_sum,
                                          bf16* dst, long out_stride, int rows_here, uint32_t stage, uint32_t spin_limit) {
    const int lane = threadIdx.x & 31;
    if (!__all_sync(0xffffffffu, MBAR_WAIT(o_done, parity))) return false;
    tc_fence_after();
    const float inv = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
    float o[D];
#pragma unroll
    for (int c = 0; c < D / 32; ++c) tmem_ld32(o_addr + c * 32, o + c * 32);
    tmem_wait_ld();
    tc_fence_before();
    mbar_arrive(o_free);                                   // the rows are in registers: the tensor cores may have the buffer
#pragma unroll
    for (int c = 0; c < D / 64; ++c) {
#pragma unroll
        for (int e = 0; e < 64; e += 8) {
            const float* v = o + c * 64 + e;
            uint4 w;
            w.x = ft_pack(v[0] * inv, v[1] * inv);
            w.y = ft_pack(v[2] * inv, v[3] * inv);
            w.z = ft_pack(v[4] * inv, v[5] * inv);
            w.w = ft_pack(v[6] * inv, v[7] * inv);
            sts128(stage + lane * 128 + (((e >> 3) ^ (lane & 7)) << 4), w);
        }
        __syncwarp();
        uint4 w[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int row = k * 4 + (lane >> 3);
            w[k] = lds128(stage + row * 128 + (((lane & 7) ^ (row & 7)) << 4));
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int row = k * 4 + (lane >> 3);
            if (row < rows_here) *reinterpret_cast<uint4*>(dst + (size_t)row * out_stride + c * 64 + (lane & 7) * 8) = w[k];
        }
        __syncwarp();
    }
    return true;
}

// What the producer tells the other warps about a work item (one per Q buffer).
struct FtItem {
    int n_tiles;      // key tiles of the item; 0: there is no further item
    int j_beg;        // first key tile
    int p0;           // position of the item's first token
    int seq_hi;       // last position the cache holds for the sequence
    int row0;         // row of the item's first token in q and out
    int rows;         // tokens of the item that exist (at most FT_ROWS)
    int head;
    int pad;
};

template <int D>
__global__ void __launch_bounds__(FT_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, long out_stride,
                            const int* __restrict__ block_table, int table_stride, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ seq_slot, const int* __restrict__ seq_start, int n_seqs, int max_tiles,
                            int n_q, int n_kv, int window, float scale_log2, uint32_t v_lbo, uint32_t v_sbo,
                            int* __restrict__ status, int* __restrict__ counters, TcWaits waits) {
    const uint32_t spin_limit = waits.spin_limit;
    constexpr int BOXES = D / 64;
    constexpr int TILE_BYTES = BOXES * FT_BOX_BYTES;       // a Q tile, a K tile or a V tile
    constexpr int PAGE_BYTES = FT_PAGE * 128;              // one page's rows inside a box
    constexpr int S_COLS = FT_KEYS;                        // columns of one S buffer
    constexpr int O_COL = 2 * S_COLS;                      // the two O buffers behind the two S buffers
    constexpr uint32_t FULL = 0xffffffffu;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_smem = smem;                           // [2] items
    unsigned char* k_smem = q_smem + 2 * TILE_BYTES;        // [2] stages
    unsigned char* v_smem = k_smem + 2 * TILE_BYTES;        // [2] stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + 2 * TILE_BYTES);
    uint64_t* q_full = bars;          // [2] the item's record is written and its Q tile has landed
    uint64_t* q_empty = bars + 2;     // [2] the item's products with Q are done and every warp has read its record
    uint64_t* k_full = bars + 4;      // [2]
    uint64_t* k_empty = bars + 6;     // [2]
    uint64_t* v_full = bars + 8;      // [2]
    uint64_t* v_empty = bars + 10;    // [2]
    uint64_t* s_full = bars + 12;     // [2]
    uint64_t* p_full = bars + 14;     // [2]
    uint64_t* o_tile = bars + 16;     // every P V product, one phase per tile
    uint64_t* o_done = bars + 17;     // [2] an item's last P V product
    uint64_t* o_free = bars + 19;     // [2] the softmax warps have read the item's O
    uint64_t* tail_bar = bars + 21;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
    volatile int* s_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile FtItem* items = reinterpret_cast<volatile FtItem*>(tmem_slot + 2);     // [2]
    int4* seq_meta = reinterpret_cast<int4*>(smem + 6 * TILE_BYTES + 512);          // [FT_META_SEQS]
    unsigned char* stage_smem = reinterpret_cast<unsigned char*>(seq_meta + FT_META_SEQS);   // [4 warps][32 rows][128 bytes]
    const bool meta_in_smem = n_seqs <= FT_META_SEQS;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&q_full[s], 1);
            mbar_init(&q_empty[s], 1 + FT_ROWS / 32);
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], FT_ROWS);
            mbar_init(&o_done[s], 1);
            mbar_init(&o_free[s], FT_ROWS);
        }
        mbar_init(o_tile, 1);
        mbar_init(tail_bar, 1);
        *s_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    // every sequence's slot, first row, number of new tokens and first position (written before
    // the step's first kernel began, so they may be read ahead of the wait)
    if (meta_in_smem)
        for (int q = threadIdx.x; q < n_seqs; q += FT_THREADS) {
            const int t0 = cu_seqlens[q];
            seq_meta[q] = make_int4(seq_slot[q], t0, cu_seqlens[q + 1] - t0, seq_start[q]);
        }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();
    pdl_wait();

    if (warp == 4 && waits.hold_producer) {
        // the probe of the time-out path: no item is drawn and no copy issued, so every other role's
        // first wait runs out
    } else if (warp == 4) {
        // ---------------------------------------------------------------- TMA producer
        const int per_level = n_seqs * n_q;
        const int total = max_tiles * per_level;
        auto meta_of = [&](int seq) -> int4 {              // slot, first row, new tokens, first position
            if (meta_in_smem) return seq_meta[seq];
            const int t0 = cu_seqlens[seq];
            return make_int4(seq_slot[seq], t0, cu_seqlens[seq + 1] - t0, seq_start[seq]);
        };
        // Items in the order: token tiles from the last one down (the longest first, so that the
        // short ones fill the tail), sequences, heads.  Tickets come from a counter that all blocks
        // share; an item is prepared (its sequence's numbers, the page ids of its first key tile)
        // while the last tiles of the item before it are loaded.
        struct Prep {
            int have, head, kvh, tok0, slot, t0, nt, start, j_beg, n_tiles, pg0, pg1;
        };
        int drawn = 0;                                     // lane 0: the ticket drawn last
        auto draw = [&]() {
            if (lane == 0) drawn = atomicAdd(&counters[0], 1);
        };
        auto page_of = [&](int slot, int idx) -> int {
            return idx < table_stride ? block_table[(size_t)slot * table_stride + idx] : -1;
        };
        auto prepare = [&]() -> Prep {                     // takes the ticket drawn before, draws on while items do not exist
            Prep p = {};
            for (;; draw()) {
                const int v = __shfl_sync(FULL, drawn, 0);
                if (v >= total) return p;
                const int lvl = v / per_level, rem = v - lvl * per_level;
                const int seq = rem / n_q;
                const int4 m = meta_of(seq);
                p.tok0 = (max_tiles - 1 - lvl) * FT_ROWS;
                if (m.x < 0 || p.tok0 >= m.z) continue;
                p.have = 1;
                p.head = rem - seq * n_q;
                p.kvh = p.head / (n_q / n_kv);
                p.slot = m.x, p.t0 = m.y, p.nt = m.z, p.start = m.w;
                const int p0 = p.start + p.tok0;                                      // position of the item's first token
                const int hi_block = p.start + min(p.tok0 + FT_ROWS - 1, p.nt - 1);
                const int lo_block = window > 0 ? max(0, p0 - window + 1) : 0;
                p.j_beg = lo_block / FT_KEYS;
                p.n_tiles = hi_block / FT_KEYS - p.j_beg + 1;                          // key tiles
                p.pg0 = page_of(p.slot, 2 * p.j_beg);
                p.pg1 = page_of(p.slot, 2 * p.j_beg + 1);
                return p;
            }
        };
        // Hands an item to the other warps: waits for its Q buffer, writes its record and loads its
        // Q tile -- or, when there is no further item, a record that says so.
        auto announce = [&](int it, const Prep& p) -> bool {
            const int qi = it & 1;
            int ok = 1;
            if (lane == 0) {
                if (it >= 2 && !MBAR_WAIT(&q_empty[qi], ((uint32_t)(it >> 1) & 1) ^ 1)) ok = 0;
                if (ok && !p.have) {
                    items[qi].n_tiles = 0;
                    mbar_arrive(&q_full[qi]);
                } else if (ok) {
                    items[qi].n_tiles = p.n_tiles;
                    items[qi].j_beg = p.j_beg;
                    items[qi].p0 = p.start + p.tok0;
                    items[qi].seq_hi = p.start + p.nt - 1;
                    items[qi].row0 = p.t0 + p.tok0;
                    items[qi].rows = p.nt - p.tok0;
                    items[qi].head = p.head;
                    mbar_expect_tx(&q_full[qi], TILE_BYTES);
                    for (int c = 0; c < BOXES; ++c)
                        tma_load_2d(q_smem + (size_t)qi * TILE_BYTES + c * FT_BOX_BYTES, &map_q, p.head * D + c * 64,
                                    p.t0 + p.tok0, &q_full[qi]);
                }
            }
            return __shfl_sync(FULL, ok, 0) != 0;
        };
        draw();
        Prep cur = prepare(), nxt = {};
        uint32_t g = 0, tail_phase = 0;                    // g counts key tiles over all items
        bool failed = !announce(0, cur);
        for (int it = 0; !failed && cur.have; ++it, cur = nxt) {
            int ok = 1;
            const int kvh = cur.kvh, slot = cur.slot, j_beg = cur.j_beg, n_tiles = cur.n_tiles;
            const int seq_hi = cur.start + cur.nt - 1;                          // last position the cache holds
            int pg_next[2] = {cur.pg0, cur.pg1};
            for (int i = 0; i < n_tiles; ++i, ++g) {
                const int j = j_beg + i, st = g & 1;
                const uint32_t ph = (g >> 1) & 1;
                const int pg[2] = {pg_next[0], pg_next[1]};
                if (i + 1 < n_tiles) {                     // the next tile's page ids travel while this tile is handled
                    pg_next[0] = page_of(slot, 2 * j + 2);
                    pg_next[1] = page_of(slot, 2 * j + 3);
                }
                const int n_have = (pg[0] >= 0) + (pg[1] >= 0);
                unsigned char* kt = k_smem + (size_t)st * TILE_BYTES;
                unsigned char* vt = v_smem + (size_t)st * TILE_BYTES;
                if (lane == 0) {
                    if (g >= 2 && !MBAR_WAIT(&k_empty[st], ph ^ 1)) ok = 0;
                    if (ok) {
                        mbar_expect_tx(&k_full[st], n_have * BOXES * PAGE_BYTES);
                        for (int h = 0; h < 2; ++h)
                            if (pg[h] >= 0)
                                for (int c = 0; c < BOXES; ++c)
                                    tma_load_2d(kt + c * FT_BOX_BYTES + h * PAGE_BYTES, &map_k, c * 64,
                                                (pg[h] * n_kv + kvh) * FT_PAGE, &k_full[st]);
                        if (g >= 2 && !MBAR_WAIT(&v_empty[st], ph ^ 1)) ok = 0;
                    }
                }
                ok = __shfl_sync(FULL, ok, 0);
                if (!ok) { failed = true; break; }
                if (__shfl_sync(FULL, *s_flag, 0)) { failed = true; break; }
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
                        if (!MBAR_WAIT(tail_bar, tail_phase)) ok = 0;
                    }
                    if (n_have > 0) tail_phase ^= 1;
                    ok = __shfl_sync(FULL, ok, 0);
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
                // The next item is drawn late, so that blocks that are ahead take more of what is
                // left, but early enough to hide the ticket's and the Q tile's way: the ticket
                // behind the third-last tile, the item itself behind the second-last one.
                if (i == max(0, n_tiles - 3)) draw();
                if (i == max(0, n_tiles - 2)) {
                    nxt = prepare();
                    if (!announce(it + 1, nxt)) { failed = true; break; }
                }
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
            // Descriptors of the buffers' first bytes; a step inside a buffer adds its offset / 16 to
            // the address field (the low 14 bits, which no buffer of this block overflows).
            // (the second buffer of a pair lies TILE_BYTES behind the first)
            const uint64_t q_desc = umma_desc_sw128(smem_u32(q_smem)), k_desc = umma_desc_sw128(smem_u32(k_smem));
            const uint64_t v_desc = umma_desc_mn_sw128(smem_u32(v_smem), v_lbo, v_sbo);
            constexpr uint64_t SECOND = TILE_BYTES >> 4;
            auto issue_qk = [&](int qi, uint32_t gt) {          // S[gt & 1] = Q(item) K(tile gt)^T
                const uint64_t qd = q_desc + (qi ? SECOND : 0), kd = k_desc + ((gt & 1) ? SECOND : 0);
                const uint32_t s_addr = tmem_base + (gt & 1) * S_COLS;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (uint32_t)(kk >> 2) * FT_BOX_BYTES + (uint32_t)(kk & 3) * 32;
                    umma_bf16(s_addr, qd + (off >> 4), kd + (off >> 4), idesc_s, kk > 0);
                }
                umma_commit(&s_full[gt & 1]);
                umma_commit(&k_empty[gt & 1]);
            };
            uint32_t g = 0;
            bool ok = MBAR_WAIT(&q_full[0], 0);
            int n_cur = ok ? items[0].n_tiles : 0;
            if (ok && n_cur > 0) {
                ok = MBAR_WAIT(&k_full[0], 0);
                if (ok) {
                    tc_fence_after();
                    issue_qk(0, 0);
                    if (n_cur == 1) umma_commit(&q_empty[0]);
                }
            }
            for (int it = 0; ok && n_cur > 0 && !*s_flag; ++it) {
                const int qi = it & 1;
                const uint32_t o_addr = tmem_base + O_COL + (uint32_t)qi * D;
                int n_next = 0;
                for (int i = 0; i < n_cur; ++i, ++g) {
                    const uint32_t b = g & 1, ph = (g >> 1) & 1;
                    // the next tile's scores go ahead of this tile's P V: the softmax of the next
                    // tile then runs while the tensor cores work on this one
                    if (i + 1 < n_cur) {
                        if (!MBAR_WAIT(&k_full[b ^ 1], ((g + 1) >> 1) & 1)) { ok = false; break; }
                        tc_fence_after();
                        issue_qk(qi, g + 1);
                        if (i + 2 == n_cur) umma_commit(&q_empty[qi]);
                    } else {
                        // the item's last tile: the first tile of the next item, if there is one
                        if (!MBAR_WAIT(&q_full[qi ^ 1], (uint32_t)((it + 1) >> 1) & 1)) { ok = false; break; }
                        n_next = items[qi ^ 1].n_tiles;
                        if (n_next > 0) {
                            if (!MBAR_WAIT(&k_full[b ^ 1], ((g + 1) >> 1) & 1)) { ok = false; break; }
                            tc_fence_after();
                            issue_qk(qi ^ 1, g + 1);
                            if (n_next == 1) umma_commit(&q_empty[qi ^ 1]);
                        }
                    }
                    if (!MBAR_WAIT(&p_full[b], ph) || !MBAR_WAIT(&v_full[b], ph)) { ok = false; break; }
                    // the item before the last one had this O buffer: its rows must have been read
                    if (i == 0 && it >= 2 && !MBAR_WAIT(&o_free[qi], ((uint32_t)(it >> 1) & 1) ^ 1)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t vd = v_desc + (b ? SECOND : 0);
                    const uint32_t p_addr = tmem_base + b * S_COLS;
#pragma unroll
                    for (int kk = 0; kk < FT_KEYS / 16; ++kk)       // 16 keys per step: 8 columns of packed P, 2048 bytes of V
                        umma_bf16_a_tmem(o_addr, p_addr + kk * 8, vd + (uint64_t)(kk * 2048 >> 4), idesc_o, (i > 0 || kk > 0));
                    umma_commit(&v_empty[b]);
                    umma_commit(o_tile);
                    if (i + 1 == n_cur) umma_commit(&o_done[qi]);
                }
                if (!ok) break;
                n_cur = n_next;
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
        bool ok = true, timed_out = false;
        // The rows of an item's O are read, divided by the sums and stored one tile into the next
        // item, when the tensor cores already have that tile's scores and the next tile's products.
        bool pending = false;
        int e_it = 0, e_row0 = 0, e_rows = 0, e_head = 0;
        float e_l = 0.0f;
        auto write_out = [&]() -> bool {
            return ft_write_out<D>(&o_done[e_it & 1], (uint32_t)(e_it >> 1) & 1, &o_free[e_it & 1],
                                   lane_base + O_COL + (uint32_t)(e_it & 1) * D, e_l,
                                   out + (size_t)(e_row0 + warp * 32) * out_stride + (size_t)e_head * D, out_stride,
                                   e_rows - warp * 32, smem_u32(stage_smem) + warp * 4096, spin_limit);
        };
        uint32_t g = 0;
        // every wait's outcome is agreed on by the whole warp: the tensor-memory accesses are warp-wide
        for (int it = 0; ok; ++it) {
            const int qi = it & 1;
            if (!__all_sync(FULL, MBAR_WAIT(&q_full[qi], (uint32_t)(it >> 1) & 1))) { ok = false; timed_out = true; break; }
            const int n_tiles = items[qi].n_tiles, j_beg = items[qi].j_beg, p0 = items[qi].p0, seq_hi = items[qi].seq_hi;
            const int row0 = items[qi].row0, rows = items[qi].rows, head = items[qi].head;
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_empty[qi]);
            if (n_tiles == 0) break;
            const uint32_t o_addr = lane_base + O_COL + (uint32_t)qi * D;
            const int pos_r = min(p0 + r, seq_hi);
            const int lo_r = window > 0 ? max(0, pos_r - window + 1) : 0;
            float m_used = -INFINITY, l_run = 0.0f;
            for (int i = 0; i < n_tiles; ++i, ++g) {
                if (__any_sync(FULL, *s_flag != 0)) { ok = false; break; }
                const int j = j_beg + i;
                const uint32_t b = g & 1, ph = (g >> 1) & 1;
                if (!__all_sync(FULL, MBAR_WAIT(&s_full[b], ph))) { ok = false; timed_out = true; break; }
                tc_fence_after();
                float s[FT_KEYS];
                const uint32_t s_addr = lane_base + b * S_COLS;
#pragma unroll
                for (int c = 0; c < FT_KEYS / 32; ++c) tmem_ld32(s_addr + c * 32, s + c * 32);
                tmem_wait_ld();
                const int key0 = j * FT_KEYS;
                const bool masked = key0 + FT_KEYS - 1 > p0 || key0 + FT_KEYS - 1 > seq_hi ||
                                    (window > 0 && key0 < p0 + FT_ROWS - 1 - window + 1);
                if (masked) {
                    // keep lo <= index <= hi; by groups of 32 keys, so that a warp passes over the
                    // groups that all its rows keep whole (on the diagonal: those left of its rows)
                    const int hi = pos_r - key0, lo = lo_r - key0;
#pragma unroll
                    for (int c = 0; c < FT_KEYS / 32; ++c) {
                        if (__all_sync(FULL, c * 32 + 31 <= hi && c * 32 >= lo)) continue;
#pragma unroll
                        for (int e = c * 32; e < c * 32 + 32; ++e) s[e] = (e > hi || e < lo) ? -INFINITY : s[e];
                    }
                }
                float mx = s[0];
#pragma unroll
                for (int e = 1; e < FT_KEYS; ++e) mx = fmaxf(mx, s[e]);
                // raise the running maximum only when a score would otherwise exceed 2^8 after the shift
                const bool raise = mx > -INFINITY && (m_used == -INFINITY || (mx - m_used) * scale_log2 > FT_RESCALE_ABOVE);
                if (__any_sync(FULL, raise && i > 0)) {
                    const float m_new = raise ? mx : m_used;
                    const float f = (raise && m_used > -INFINITY) ? ft_exp2((m_used - m_new) * scale_log2) : 1.0f;
                    if (!__all_sync(FULL, MBAR_WAIT(o_tile, (g - 1) & 1))) {     // O holds the item's tiles 0 .. i-1
                        ok = false;
                        timed_out = true;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        float o[32];
                        uint32_t ou[32];
                        tmem_ld32(o_addr + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) ou[e] = __float_as_uint(o[e] * f);
                        tmem_st32(o_addr + c * 32, ou);
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
                if (i == 0 && pending) {
                    pending = false;
                    if (!write_out()) { ok = false; timed_out = true; break; }
                }
            }
            if (!ok) break;
            pending = true;
            e_it = it, e_row0 = row0, e_rows = rows, e_head = head, e_l = l_run;
        }
        if (ok && pending && !write_out()) timed_out = true;
        if (timed_out && lane == 0) {
            atomicOr(status, BFI_STATUS_TIMEOUT);
            *s_flag = 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*s_flag && warp == 4 && lane == 0) {
        // a wait ran out: give outstanding TMA writes a bounded time to land
        for (int s = 0; s < 2; ++s) {
            MBAR_WAIT(&q_full[s], 0), MBAR_WAIT(&q_full[s], 1);
            MBAR_WAIT(&k_full[s], 0), MBAR_WAIT(&k_full[s], 1);
            MBAR_WAIT(&v_full[s], 0), MBAR_WAIT(&v_full[s], 1);
        }
        MBAR_WAIT(tail_bar, 0), MBAR_WAIT(tail_bar, 1);
    }
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    // the last block to finish puts the ticket counter back for the next launch
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&counters[1], 1) == (int)gridDim.x - 1) {
            counters[0] = 0;
            counters[1] = 0;
            __threadfence();
        }
    }
    BFI_TRACE_END();
}

template <int D>
static int launch_prefill_tc(const void* qkv, long q_stride, void* out, long out_stride, const void* k_pages,
                             const void* v_pages, long n_pages, const int* block_table, int table_stride,
                             const int* cu_seqlens, const int* seq_slot, const int* seq_start, int n_seqs, long n_tokens,
                             int max_seq_tokens, int n_q, int n_kv, int window, float scale, int* status,
                             cudaStream_t stream, TcWaits waits) {
    CUtensorMap mq, mk, mv;
    int rc = bfi_tensor_map_bf16(qkv, n_tokens, (long)n_q * D, q_stride, FT_ROWS, &mq);
    if (rc) return rc;
    rc = bfi_tensor_map_bf16(k_pages, n_pages * n_kv * FT_PAGE, D, D, FT_PAGE, &mk);
    if (rc) return rc;
    rc = bfi_tensor_map_bf16(v_pages, n_pages * n_kv * FT_PAGE, D, D, FT_PAGE, &mv);
    if (rc) return rc;
    constexpr int TILE_BYTES = (D / 64) * FT_BOX_BYTES;
    // at least half an SM's shared memory, so that two blocks never share one SM's tensor memory
    const size_t tiles = (size_t)6 * TILE_BYTES + 1024 + 512 + FT_META_SEQS * sizeof(int4) + 4 * 4096;
    const size_t smem = tiles > 120 * 1024 ? tiles : 120 * 1024;
    auto kernel = attention_prefill_tc_kernel<D>;
    static bool configured = false;
    const int n_sm = bfi_sm_count();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return bfi_fail("attention_prefill_tcgen05: cannot reserve %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
        configured = true;
    }
    const unsigned lbo = FT_BOX_BYTES;      // leading byte offset: between the two 64-wide halves of the head
    const unsigned sbo = 1024;              // stride byte offset: between groups of 8 keys
    const int max_tiles = (max_seq_tokens + FT_ROWS - 1) / FT_ROWS;
    const long items = (long)max_tiles * n_seqs * n_q;
    dim3 grid((unsigned)(items < n_sm ? items : n_sm));      // one block per SM, each drawing items until none is left
    bfi_launch(kernel, grid, dim3(FT_THREADS), smem, stream, mq, mk, mv, (bf16*)out, out_stride, block_table, table_stride,
               cu_seqlens, seq_slot, seq_start, n_seqs, max_tiles, n_q, n_kv, window, scale * 1.4426950408889634f,
               (uint32_t)lbo, (uint32_t)sbo, status, status + 1, waits);
    return bfi_check_launch("attention_prefill_tcgen05");
}

// qkv [n_tokens, >= n_q*d] with the step's query heads (already normalised and rotated), the
// cache pages [n_pages, n_kv, 64, d] holding every key and value up to each sequence's last new
// token.  Returns 0 on success, 1 on error, 2 when the shape is not taken (nothing launched):
// head sizes other than 64/128, or operands TMA cannot address.  `status` points at three ints,
// zero before the first call: [0] gets BFI_STATUS_TIMEOUT when a wait ran out, [1] and [2] are
// the counters of tickets drawn and blocks finished, which every launch leaves at zero again; two
// launches that may run at the same time need status words of their own.
static int attention_prefill_tc_launch(const void* qkv, long q_stride, void* out, long out_stride, const void* k_pages,
                                       const void* v_pages, long n_pages, const int* block_table, int table_stride,
                                       const int* cu_seqlens, const int* seq_slot, const int* seq_start, int n_seqs,
                                       long n_tokens, int max_seq_tokens, int n_q, int n_kv, int d, int window, float scale,
                                       int* status, cudaStream_t stream, TcWaits waits) {
    BFI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_prefill_tcgen05: %d query heads do not divide into %d kv heads",
                n_q, n_kv);
    BFI_REQUIRE(window >= 0 && status != nullptr, "attention_prefill_tcgen05: bad window or no status word");
    if (n_seqs <= 0 || max_seq_tokens <= 0) return 0;
    if (d != 64 && d != 128) return 2;
    if (q_stride % 8 != 0 || out_stride % 8 != 0 || ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15) ||
        ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || (long)((max_seq_tokens + FT_ROWS - 1) / FT_ROWS) * n_seqs * n_q > 0x3fffffffL)
        return 2;
    if (n_pages * n_kv * FT_PAGE > 0x7fffffffL) return 2;       // TMA coordinates are 32-bit
    if (d == 64)
        return launch_prefill_tc<64>(qkv, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                     cu_seqlens, seq_slot, seq_start, n_seqs, n_tokens, max_seq_tokens, n_q, n_kv, window,
                                     scale, status, stream, waits);
    return launch_prefill_tc<128>(qkv, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                  cu_seqlens, seq_slot, seq_start, n_seqs, n_tokens, max_seq_tokens, n_q, n_kv, window, scale,
                                  status, stream, waits);
}

extern "C" int bfi_attention_prefill_tcgen05_bf16(const void* qkv, long q_stride, void* out, long out_stride,
                                                  const void* k_pages, const void* v_pages, long n_pages,
                                                  const int* block_table, int table_stride, const int* cu_seqlens,
                                                  const int* seq_slot, const int* seq_start, int n_seqs, long n_tokens,
                                                  int max_seq_tokens, int n_q, int n_kv, int d, int window, float scale,
                                                  int* status, cudaStream_t stream) {
    return attention_prefill_tc_launch(qkv, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                       cu_seqlens, seq_slot, seq_start, n_seqs, n_tokens, max_seq_tokens, n_q, n_kv, d, window,
                                       scale, status, stream, tc_waits_default());
}

// For the tests of the time-out path: the same launch, but every bounded wait gives up after
// `spin_limit` polls (at most 65536 here) and, with hold_producer != 0, the producer warp draws no
// item and issues no copy, so that the first wait of every other role runs out by construction.
// The launch records BFI_STATUS_TIMEOUT in status[0], leaves the ticket counters at zero, frees its
// tensor memory and returns; `out` is not written.  No fault, no trap, nothing unbounded.
extern "C" int bfi_attention_prefill_tcgen05_bf16_wait_probe(const void* qkv, long q_stride, void* out, long out_stride,
                                                             const void* k_pages, const void* v_pages, long n_pages,
                                                             const int* block_table, int table_stride,
                                                             const int* cu_seqlens, const int* seq_slot,
                                                             const int* seq_start, int n_seqs, long n_tokens,
                                                             int max_seq_tokens, int n_q, int n_kv, int d, int window,
                                                             float scale, int* status, unsigned spin_limit,
                                                             int hold_producer, cudaStream_t stream) {
    BFI_REQUIRE(spin_limit >= 1 && spin_limit <= 65536, "attention_prefill_tcgen05 wait probe: spin limit %u outside 1..65536",
                spin_limit);
    return attention_prefill_tc_launch(qkv, q_stride, out, out_stride, k_pages, v_pages, n_pages, block_table, table_stride,
                                       cu_seqlens, seq_slot, seq_start, n_seqs, n_tokens, max_seq_tokens, n_q, n_kv, d, window,
                                       scale, status, stream, TcWaits{spin_limit, hold_producer ? 1 : 0});
}

BFI_TRACE_EXPORT(attention_prefill_tcgen05)
