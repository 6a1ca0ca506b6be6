// Choosing the next token from float32 logits on the device: greedy, and temperature sampling
// with the reference's penalties and min-p cut, one block per row.
//
// Reference (crates/bfi-runtime/src/sample.rs):
//   argmax            :429-439  strict '>' scan from index 0, so the lowest index among equal maxima wins
//   repeat penalty    :345-357  every id seen so far: logit > 0 ? logit / pen : logit * pen
//   presence penalty  :359-367  logit -= pen for every seen id, after the repeat penalty
//   temperature       :369-390  <= 0 means argmax; else logits / T, max-subtracted softmax
//   min-p             :411-424  keep p >= min_p * p_max
//   draw              :312-323  r = u * sum(kept); the first kept id, in vocabulary order, whose running sum reaches r
//   top-k             :392-395  stable sort by descending probability, keep the first k
//   top-p             :397-409  the same order; keep through the first position whose running sum reaches top_p
// Top-k and top-p do not sort here: the kept set is a prefix of the order (probability descending,
// index ascending), and a prefix is found by a radix descent over the probabilities' bit patterns
// (sample_sorted_rows_kernel below); the draw, which the reference makes in that same order, is a
// second descent.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_ITEMS 4

struct ArgBest {
    float v;
    int i;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ ArgBest block_argmax(ArgBest mine, ArgBest* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other;
        other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
        mine = better(mine, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    if (warp == 0) {
        ArgBest t;
        t.v = -INFINITY;
        t.i = 0x7fffffff;
        if (lane < n_warps) t = scratch[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgBest other;
            other.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            other.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, other);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Applies the penalties for one seen id list to a row held in global memory (work row).
__device__ __forceinline__ float penalised(float v, float repeat_penalty, float presence_penalty) {
    if (repeat_penalty != 1.0f) v = v > 0.0f ? v / repeat_penalty : v * repeat_penalty;
    return v - presence_penalty;
}

// One block per row.
//   logits        [rows, stride] float32 (never modified)
//   work          [rows, vocab] float32 scratch, needed only when a row has seen ids (else may be null)
//   seen, seen_cu ids seen by each row, every id at most once per row; seen_cu [rows+1] offsets (null: none)
//   temperature, u per row.  u in [0, 1).
//   out           [rows] int32
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, long stride, float* __restrict__ work, int vocab,
                   const int* __restrict__ seen, const int* __restrict__ seen_cu, const float* __restrict__ temperature,
                   const float* __restrict__ u_draw, float repeat_penalty, float presence_penalty, float min_p,
                   int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ ArgBest abest[33];
    __shared__ float fscratch[33];
    __shared__ float warp_tot[32];
    __shared__ int found;
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * stride;

    // ---- penalties: copy the row and edit the seen ids
    const int n_seen = seen_cu ? seen_cu[row + 1] - seen_cu[row] : 0;
    if (n_seen > 0 && (repeat_penalty != 1.0f || presence_penalty != 0.0f)) {
        float* w = work + (size_t)row * vocab;
        for (int j = threadIdx.x; j < vocab; j += blockDim.x) w[j] = x[j];
        __syncthreads();
        const int* ids = seen + seen_cu[row];
        for (int s = threadIdx.x; s < n_seen; s += blockDim.x) {
            const int id = ids[s];
            if (id >= 0 && id < vocab) w[id] = penalised(w[id], repeat_penalty, presence_penalty);
        }
        __syncthreads();
        x = w;
    }

    // ---- maximum and its lowest index
    ArgBest mine;
    mine.v = -INFINITY;
    mine.i = 0x7fffffff;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float v = x[j];
        if (v > mine.v) {  // strict: within a thread indices ascend, so the first maximum stays
            mine.v = v;
            mine.i = j;
        }
    }
    const ArgBest best = block_argmax(mine, abest);
    const int arg = best.i == 0x7fffffff ? 0 : best.i;
    const float temp = temperature[row];
    if (!(temp > 0.0f)) {
        if (threadIdx.x == 0) out[row] = arg;
        return;
    }

    // ---- softmax denominators.  e_j = exp((x_j - max) / T); p_j = e_j / sum; p_max = 1 / sum.
    const float inv_t = 1.0f / temp;
    const float mx = best.v;
    float part = 0.0f, kept = 0.0f;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float e = expf((x[j] - mx) * inv_t);
        part += e;
        if (e >= min_p) kept += e;   // p_j >= min_p * p_max  <=>  e_j >= min_p
    }
    const float total = block_sum(part, fscratch);
    const float total_kept = min_p > 0.0f ? block_sum(kept, fscratch) : total;
    if (!(total > 0.0f) || !(total_kept > 0.0f)) {
        if (threadIdx.x == 0) out[row] = arg;
        return;
    }
    const float r = u_draw[row] * total_kept;

    // ---- inverse CDF in vocabulary order: chunks of SAMPLE_THREADS * SAMPLE_ITEMS consecutive ids
    if (threadIdx.x == 0) found = 0x7fffffff;
    __syncthreads();
    float running = 0.0f;
    int last_kept = -1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < vocab; base += SAMPLE_THREADS * SAMPLE_ITEMS) {
        float e[SAMPLE_ITEMS];
        float local = 0.0f;
        const int j0 = base + threadIdx.x * SAMPLE_ITEMS;
#pragma unroll
        for (int k = 0; k < SAMPLE_ITEMS; ++k) {
            const int j = j0 + k;
            float v = 0.0f;
            if (j < vocab) {
                v = expf((x[j] - mx) * inv_t);
                if (v < min_p) v = 0.0f;
            }
            e[k] = v;
            local += v;
        }
        // exclusive prefix of `local` over the block
        float incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        float before = running;
        for (int w2 = 0; w2 < warp; ++w2) before += warp_tot[w2];
        float chunk_total = 0.0f;
        for (int w2 = 0; w2 < (SAMPLE_THREADS >> 5); ++w2) chunk_total += warp_tot[w2];
        float cum = before + (incl - local);
#pragma unroll
        for (int k = 0; k < SAMPLE_ITEMS; ++k) {
            if (e[k] > 0.0f) {
                cum += e[k];
                last_kept = j0 + k;
                if (r <= cum) {
                    atomicMin(&found, j0 + k);
                    break;
                }
            }
        }
        running += chunk_total;
        __syncthreads();
        if (found != 0x7fffffff) break;
    }
    if (found == 0x7fffffff) {
        // rounding left r above the final running sum: the last kept id, as the reference does
        const float m = block_max((float)last_kept, fscratch);
        if (threadIdx.x == 0) out[row] = m >= 0.0f ? (int)m : arg;
        return;
    }
    if (threadIdx.x == 0) out[row] = found;
}

extern "C" int bfi_sample_rows(const float* logits, long stride, float* work, int n_rows, int vocab, const int* seen,
                               const int* seen_cu, const float* temperature, const float* u_draw, float repeat_penalty,
                               float presence_penalty, float min_p, int* out, cudaStream_t stream) {
    BFI_REQUIRE(n_rows >= 0 && vocab > 0, "sample_rows: bad sizes rows=%d vocab=%d", n_rows, vocab);
    BFI_REQUIRE(stride >= vocab, "sample_rows: row stride shorter than the vocabulary");
    BFI_REQUIRE(temperature && u_draw && out && logits, "sample_rows: null argument");
    BFI_REQUIRE(vocab < (1 << 24), "sample_rows: vocabulary %d too large", vocab);
    if (seen_cu && (repeat_penalty != 1.0f || presence_penalty != 0.0f))
        BFI_REQUIRE(work != nullptr && seen != nullptr, "sample_rows: penalties need a work buffer and the seen ids");
    BFI_REQUIRE(repeat_penalty > 0.0f, "sample_rows: repeat_penalty must be positive");
    if (n_rows == 0) return 0;
    bfi_launch(sample_rows_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, stride, work, vocab, seen, seen_cu, temperature,
                                                             u_draw, repeat_penalty, presence_penalty, min_p, out);
    return bfi_check_launch("sample_rows");
}

// ------------------------------------------------------------------------------------------
// Top-k / top-p: one block per row.
//
// Order: probability descending, index ascending (the reference's stable sort).  Everything the
// reference does after the sort works on prefixes of that order: top-k keeps the first k, top-p
// keeps through the first position whose running sum reaches top_p, min-p (relative to the largest
// probability) drops a tail, and the draw returns the first position whose running sum reaches
// r = u * (sum of the kept).  A prefix is described by a boundary: a probability value v and an
// index i -- kept are p > v, and p == v with index <= i.  The boundary is found by a radix descent
// over the 32-bit patterns of the probabilities (non-negative floats order like their patterns):
// four passes of 8 bits, each a 256-bin histogram of counts and masses, walked from the top bin
// down until the count or the mass reaches its limit.  Masses are summed as 64-bit fixed point
// (p * 2^40), so the sums do not depend on the order of the additions.
// ------------------------------------------------------------------------------------------
#define SS_FIX 1099511627776.0f      // 2^40

struct Boundary {
    unsigned int value;              // bit pattern of the boundary probability
    int index;                       // last index kept among probabilities equal to it
    int all;                         // nothing is cut: every candidate lies above the boundary
};

__device__ __forceinline__ unsigned long long fix40(float p) { return (unsigned long long)(p * SS_FIX); }

__device__ __forceinline__ bool above(const Boundary& b, unsigned int bits, int j) {
    return b.all || bits > b.value || (bits == b.value && j <= b.index);
}

// The boundary of the shortest prefix (of the candidates: probabilities >= floor_bits that lie above
// `within`) whose count reaches limit_cnt or whose mass reaches limit_mass; at least one element.
__device__ Boundary radix_prefix(const float* __restrict__ p, int vocab, const Boundary& within, unsigned int floor_bits,
                                 int limit_cnt, unsigned long long limit_mass, int* h_cnt, unsigned long long* h_mass,
                                 int* s_int, unsigned long long* s_u64) {
    unsigned int prefix = 0;                       // the bits decided so far, in place
    int cnt_above = 0;
    unsigned long long mass_above = 0;
    Boundary out;
    out.value = 0;
    out.index = 0x7fffffff;
    out.all = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) {
            h_cnt[i] = 0;
            h_mass[i] = 0;
        }
        __syncthreads();
        const unsigned int hi_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
            const float v = p[j];
            const unsigned int bits = __float_as_uint(v);
            if (bits < floor_bits || !above(within, bits, j) || (bits & hi_mask) != prefix) continue;
            const int bin = (bits >> shift) & 255;
            atomicAdd(&h_cnt[bin], 1);
            atomicAdd(&h_mass[bin], fix40(v));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int found = -1;
            for (int b = 255; b >= 0; --b) {
                if (h_cnt[b] == 0) continue;
                if (cnt_above + h_cnt[b] >= limit_cnt || mass_above + h_mass[b] >= limit_mass) {
                    found = b;
                    break;
                }
                cnt_above += h_cnt[b];
                mass_above += h_mass[b];
            }
            s_int[0] = found;
            s_int[1] = cnt_above;
            s_u64[0] = mass_above;
        }
        __syncthreads();
        const int found = s_int[0];
        cnt_above = s_int[1];
        mass_above = s_u64[0];
        __syncthreads();
        if (found < 0) {                            // the limits are never reached: the prefix is everything
            out.all = 1;
            return out;
        }
        prefix |= (unsigned int)found << shift;
    }
    // among the candidates equal to the boundary value, in index order: how many are needed
    out.value = prefix;
    const unsigned long long q = fix40(__uint_as_float(prefix));
    long long need = 1;
    {
        long long by_cnt = (long long)limit_cnt - cnt_above;                    // t with cnt_above + t >= limit_cnt
        long long by_mass = 0x7fffffffffffffffLL;
        if (limit_mass != 0xffffffffffffffffULL) {
            const unsigned long long gap = limit_mass > mass_above ? limit_mass - mass_above : 0;
            by_mass = q > 0 ? (long long)((gap + q - 1) / q) : 0x7fffffffffffffffLL;
        }
        need = by_cnt < by_mass ? by_cnt : by_mass;
        if (need < 1) need = 1;
    }
    // each thread counts the equal candidates of a contiguous stretch of ids; an exclusive scan of the
    // counts tells which stretch holds the need-th one
    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int beg = min(vocab, (int)threadIdx.x * per), end = min(vocab, beg + per);
    int mine = 0;
    for (int j = beg; j < end; ++j) {
        const unsigned int bits = __float_as_uint(p[j]);
        if (bits == prefix && bits >= floor_bits && above(within, bits, j)) ++mine;
    }
    // block-wide exclusive scan through shared memory (h_cnt has 256 ints: scan warp totals there)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) h_cnt[warp] = incl;
    if (threadIdx.x == 0) s_int[2] = 0x7fffffff;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += h_cnt[w];
    before += incl - mine;
    if (mine > 0 && before < need && need <= before + mine) {
        long long seen = before;
        for (int j = beg; j < end; ++j) {
            const unsigned int bits = __float_as_uint(p[j]);
            if (bits == prefix && bits >= floor_bits && above(within, bits, j) && ++seen == need) {
                s_int[2] = j;
                break;
            }
        }
    }
    __syncthreads();
    out.index = s_int[2];                           // fewer equal candidates than needed: all of them (0x7fffffff)
    __syncthreads();
    return out;
}

//   probs  [rows, vocab] float32 scratch (the probabilities of every row are left there)
//   work   [rows, vocab] float32 scratch for rows with seen ids (may be null without penalties)
//   top_k <= 0 or >= vocab: no count limit; top_p >= 1: no mass limit
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_sorted_rows_kernel(const float* __restrict__ logits, long stride, float* __restrict__ work, float* __restrict__ probs,
                          int vocab, const int* __restrict__ seen, const int* __restrict__ seen_cu,
                          const float* __restrict__ temperature, const float* __restrict__ u_draw, float repeat_penalty,
                          float presence_penalty, int top_k, float top_p, float min_p, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ ArgBest abest[33];
    __shared__ float fscratch[33];
    __shared__ int h_cnt[256];
    __shared__ unsigned long long h_mass[256];
    __shared__ int s_int[4];
    __shared__ unsigned long long s_u64[2];
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * stride;
    float* p = probs + (size_t)row * vocab;

    // ---- the maximum of the unpenalised row: what the reference falls back to when min-p empties the set
    ArgBest mine;
    mine.v = -INFINITY;
    mine.i = 0x7fffffff;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float v = x[j];
        if (v > mine.v) {
            mine.v = v;
            mine.i = j;
        }
    }
    const ArgBest plain_best = block_argmax(mine, abest);
    __syncthreads();

    // ---- penalties: copy the row and edit the seen ids
    const int n_seen = seen_cu ? seen_cu[row + 1] - seen_cu[row] : 0;
    ArgBest best = plain_best;
    if (n_seen > 0 && (repeat_penalty != 1.0f || presence_penalty != 0.0f)) {
        float* w = work + (size_t)row * vocab;
        for (int j = threadIdx.x; j < vocab; j += blockDim.x) w[j] = x[j];
        __syncthreads();
        const int* ids = seen + seen_cu[row];
        for (int s = threadIdx.x; s < n_seen; s += blockDim.x) {
            const int id = ids[s];
            if (id >= 0 && id < vocab) w[id] = penalised(w[id], repeat_penalty, presence_penalty);
        }
        __syncthreads();
        x = w;
        mine.v = -INFINITY;
        mine.i = 0x7fffffff;
        for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
            const float v = x[j];
            if (v > mine.v) {
                mine.v = v;
                mine.i = j;
            }
        }
        best = block_argmax(mine, abest);
        __syncthreads();
    }
    const int arg = best.i == 0x7fffffff ? 0 : best.i;
    const float temp = temperature[row];
    if (!(temp > 0.0f)) {
        if (threadIdx.x == 0) out[row] = arg;
        return;
    }

    // ---- probabilities
    const float inv_t = 1.0f / temp;
    float part = 0.0f;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float e = expf((x[j] - best.v) * inv_t);
        p[j] = e;
        part += e;
    }
    const float total = block_sum(part, fscratch);
    __syncthreads();
    if (!(total > 0.0f)) {
        if (threadIdx.x == 0) out[row] = arg;
        return;
    }
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) p[j] = p[j] / total;
    __syncthreads();
    const float p_max = 1.0f / total;                                    // e of the maximum is 1

    // ---- the cuts
    Boundary everything;
    everything.value = 0;
    everything.index = 0x7fffffff;
    everything.all = 1;
    const int limit_cnt = (top_k > 0 && top_k < vocab) ? top_k : 0x7fffffff;
    const unsigned long long limit_mass = top_p < 1.0f ? fix40(fmaxf(top_p, 0.0f)) : 0xffffffffffffffffULL;
    Boundary kept = everything;
    if (limit_cnt != 0x7fffffff || limit_mass != 0xffffffffffffffffULL)
        kept = radix_prefix(p, vocab, everything, 0u, limit_cnt, limit_mass, h_cnt, h_mass, s_int, s_u64);
    unsigned int floor_bits = 0u;
    if (min_p > 0.0f) {
        const float thresh = min_p * p_max;
        if (!(p_max >= thresh)) {                                        // min_p above 1 empties the set
            if (threadIdx.x == 0) out[row] = plain_best.i == 0x7fffffff ? 0 : plain_best.i;
            return;
        }
        floor_bits = __float_as_uint(thresh);
    }

    // ---- the draw: r = u * (sum of the kept), then the first position in order whose running sum reaches r
    unsigned long long mass = 0;
    {
        unsigned long long local = 0;
        for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
            const unsigned int bits = __float_as_uint(p[j]);
            if (bits >= floor_bits && above(kept, bits, j)) local += fix40(p[j]);
        }
        if (threadIdx.x == 0) s_u64[1] = 0;
        __syncthreads();
        atomicAdd(&s_u64[1], local);
        __syncthreads();
        mass = s_u64[1];
        __syncthreads();
    }
    const double r = (double)u_draw[row] * (double)mass;
    unsigned long long r_fix = (unsigned long long)r;
    if ((double)r_fix < r) ++r_fix;                                     // running sum >= r, r rounded up to the grid
    Boundary pick = radix_prefix(p, vocab, kept, floor_bits, 0x7fffffff, r_fix, h_cnt, h_mass, s_int, s_u64);
    // the chosen id is the last element of that prefix: the largest index among the boundary value's
    // kept candidates up to pick.index, or, if everything was needed, the last element in order
    ArgBest tail;                                                        // "better" = smaller probability, then larger index
    tail.v = INFINITY;
    tail.i = -1;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float v = p[j];
        const unsigned int bits = __float_as_uint(v);
        if (bits < floor_bits || !above(kept, bits, j) || !above(pick, bits, j)) continue;
        if (v < tail.v || (v == tail.v && j > tail.i)) {
            tail.v = v;
            tail.i = j;
        }
    }
    // reduce: smallest probability, then largest index
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, tail.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, tail.i, o);
        if (ov < tail.v || (ov == tail.v && oi > tail.i)) {
            tail.v = ov;
            tail.i = oi;
        }
    }
    __syncthreads();
    if (lane == 0) abest[warp] = tail;
    __syncthreads();
    if (threadIdx.x == 0) {
        ArgBest t = abest[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (abest[w].v < t.v || (abest[w].v == t.v && abest[w].i > t.i)) t = abest[w];
        out[row] = t.i >= 0 ? t.i : arg;
    }
}

extern "C" int bfi_sample_sorted_rows(const float* logits, long stride, float* work, float* probs, int n_rows, int vocab,
                                      const int* seen, const int* seen_cu, const float* temperature, const float* u_draw,
                                      float repeat_penalty, float presence_penalty, int top_k, float top_p, float min_p,
                                      int* out, cudaStream_t stream) {
    BFI_REQUIRE(n_rows >= 0 && vocab > 0, "sample_sorted_rows: bad sizes rows=%d vocab=%d", n_rows, vocab);
    BFI_REQUIRE(stride >= vocab, "sample_sorted_rows: row stride shorter than the vocabulary");
    BFI_REQUIRE(temperature && u_draw && out && logits && probs, "sample_sorted_rows: null argument");
    BFI_REQUIRE(vocab < (1 << 24), "sample_sorted_rows: vocabulary %d too large", vocab);
    if (seen_cu && (repeat_penalty != 1.0f || presence_penalty != 0.0f))
        BFI_REQUIRE(work != nullptr && seen != nullptr, "sample_sorted_rows: penalties need a work buffer and the seen ids");
    BFI_REQUIRE(repeat_penalty > 0.0f, "sample_sorted_rows: repeat_penalty must be positive");
    if (n_rows == 0) return 0;
    bfi_launch(sample_sorted_rows_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, stride, work, probs, vocab, seen,
               seen_cu, temperature, u_draw, repeat_penalty, presence_penalty, top_k, top_p, min_p, out);
    return bfi_check_launch("sample_sorted_rows");
}

// Greedy only: out[row] = lowest index of the row maximum.
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_rows_kernel(const float* __restrict__ logits, long stride, int vocab, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ ArgBest abest[33];
    const float* x = logits + (size_t)blockIdx.x * stride;
    ArgBest mine;
    mine.v = -INFINITY;
    mine.i = 0x7fffffff;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) {
        const float v = x[j];
        if (v > mine.v) {
            mine.v = v;
            mine.i = j;
        }
    }
    const ArgBest best = block_argmax(mine, abest);
    if (threadIdx.x == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
}

// Large vocabularies: the row is cut into chunks, one block each, and a second kernel picks among
// the chunks' winners; ties still go to the lowest index.
#define ARGMAX_CHUNK 8192

__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float* __restrict__ logits, long stride, int vocab, int n_chunks, float* __restrict__ best_v,
                     int* __restrict__ best_i) {
    pdl_trigger();
    pdl_wait();
    __shared__ ArgBest abest[33];
    const int row = blockIdx.y, chunk = blockIdx.x;
    const float* x = logits + (size_t)row * stride;
    const int beg = chunk * ARGMAX_CHUNK, end = min(vocab, beg + ARGMAX_CHUNK);
    ArgBest mine;
    mine.v = -INFINITY;
    mine.i = 0x7fffffff;
    for (int j = beg + threadIdx.x; j < end; j += blockDim.x) {
        const float v = x[j];
        if (v > mine.v) {
            mine.v = v;
            mine.i = j;
        }
    }
    const ArgBest best = block_argmax(mine, abest);
    if (threadIdx.x == 0) {
        best_v[(size_t)row * n_chunks + chunk] = best.v;
        best_i[(size_t)row * n_chunks + chunk] = best.i;
    }
}

__global__ void __launch_bounds__(64)
argmax_pick_kernel(const float* __restrict__ best_v, const int* __restrict__ best_i, int n_chunks, int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ ArgBest abest[33];
    const int row = blockIdx.x;
    ArgBest mine;
    mine.v = -INFINITY;
    mine.i = 0x7fffffff;
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
        ArgBest o;
        o.v = best_v[(size_t)row * n_chunks + c];
        o.i = best_i[(size_t)row * n_chunks + c];
        mine = better(mine, o);
    }
    const ArgBest best = block_argmax(mine, abest);
    if (threadIdx.x == 0) out[row] = best.i == 0x7fffffff ? 0 : best.i;
}

// `scratch` (optional) holds 2 * n_rows * ceil(vocab / 8192) 4-byte values; with it, large
// vocabularies are searched by many blocks per row.
extern "C" int bfi_argmax_rows(const float* logits, long stride, int n_rows, int vocab, int* out, void* scratch,
                               long scratch_values, cudaStream_t stream) {
    BFI_REQUIRE(n_rows >= 0 && vocab > 0, "argmax_rows: bad sizes rows=%d vocab=%d", n_rows, vocab);
    BFI_REQUIRE(stride >= vocab, "argmax_rows: row stride shorter than the vocabulary");
    if (n_rows == 0) return 0;
    const int n_chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    if (scratch != nullptr && n_chunks > 1 && scratch_values >= 2L * n_rows * n_chunks && n_rows <= 65535) {
        float* bv = reinterpret_cast<float*>(scratch);
        int* bi = reinterpret_cast<int*>(scratch) + (size_t)n_rows * n_chunks;
        bfi_launch(argmax_chunks_kernel, dim3(n_chunks, n_rows), dim3(256), 0, stream, logits, stride, vocab, n_chunks, bv, bi);
        int rc = bfi_check_launch("argmax_chunks");
        if (rc) return rc;
        bfi_launch(argmax_pick_kernel, dim3(n_rows), dim3(64), 0, stream, (const float*)bv, (const int*)bi, n_chunks, out);
        return bfi_check_launch("argmax_pick");
    }
    bfi_launch(argmax_rows_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, stride, vocab, out);
    return bfi_check_launch("argmax_rows");
}

BFI_TRACE_EXPORT(sampling)
