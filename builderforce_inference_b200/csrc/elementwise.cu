// Memory-bound row kernels: embedding gather, RMS norm, SiLU*mul, and the fused
// q/k-norm + rotation + cache write that follows the QKV projection.
//
// Formulas (reference, Rust, f32 throughout):
//   embedding   crates/bfi-core/src/cpu.rs:402-438
//   RMS norm    crates/bfi-core/src/cpu.rs:92-122   y = x * rsqrt(mean(x^2) + eps) * w
//   SiLU*mul    crates/bfi-core/src/cpu.rs:169-180, 708-720
//   rotation    crates/bfi-core/src/cpu.rs:650-670  (NEOX: i pairs with i + n_rot/2)
//   per-head q/k norm before the rotation, then the cache append:
//               crates/bfi-models/src/qwen3.rs:228-234
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :]   (out is the float32 residual stream)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ out, int width, int vocab, int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, BFI_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < width; j += blockDim.x) o[j] = 0.0f;
        return;
    }
    const T* row = table + (size_t)id * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) o[j] = to_f32(row[j]);
}

extern "C" int bfi_embed_rows(const void* table, int table_dtype, const int* ids, float* out,
                              int n_tokens, int width, int vocab, int* status, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(table_dtype), "embed_rows: unknown table dtype code %d", table_dtype);
    BFI_REQUIRE(n_tokens >= 0 && width > 0 && vocab > 0, "embed_rows: bad sizes tokens=%d width=%d vocab=%d",
                n_tokens, width, vocab);
    if (n_tokens == 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == BFI_F32)
        bfi_launch(embed_rows_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, ids, out, width, vocab, status);
    else
        bfi_launch(embed_rows_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, (const bf16*)table, ids, out, width, vocab, status);
    return bfi_check_launch("embed_rows");
}

// ------------------------------------------------------------------------------------------
// RMS norm over rows of the float32 residual stream (optionally a gathered subset of rows).
// One block per output row; the sum of squares and the scale are float32.
// ------------------------------------------------------------------------------------------
template <typename TX>
__global__ void rmsnorm_kernel(const TX* __restrict__ x, long x_stride, const int* __restrict__ rows,
                               const void* __restrict__ w, int w_dtype, void* __restrict__ out,
                               int out_dtype, long out_stride, int width, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const long src = rows ? (long)rows[r] : (long)r;
    const TX* xr = x + src * x_stride;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = to_f32(xr[j]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    const size_t obase = (size_t)r * out_stride;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = to_f32(xr[j]) * scale * load_as_f32(w, w_dtype, j);
        store_from_f32(out, out_dtype, obase + j, v);
    }
}

// Single pass for float32 rows whose width is a multiple of 4 and at most 4 * VPT * THREADS: the
// row stays in registers between the sum of squares and the scaling, so it is read once.  Few rows
// (a decode step) take 256 threads a row; many rows (a prompt) take 128, so that twice as many rows
// are in flight on an SM and the whole prompt is resident at once.
template <int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS)
rmsnorm_regs_kernel(const float* __restrict__ x, long x_stride, const int* __restrict__ rows,
                    const void* __restrict__ w, int w_dtype, void* __restrict__ out, int out_dtype,
                    long out_stride, int width, float eps) {
    pdl_trigger();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int n4 = width >> 2;
    // the weights and the row index do not come from the kernel before this one: fetched before the wait
    const long src = rows ? (long)rows[r] : (long)r;
    float4 wv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int j = i * THREADS + threadIdx.x;
        const int c = j * 4;
        wv[i] = j < n4 ? make_float4(load_as_f32(w, w_dtype, c), load_as_f32(w, w_dtype, c + 1), load_as_f32(w, w_dtype, c + 2),
                                     load_as_f32(w, w_dtype, c + 3))
                       : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    const float4* xr = reinterpret_cast<const float4*>(x + src * x_stride);
    float4 v[VPT];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int j = i * THREADS + threadIdx.x;
        v[i] = j < n4 ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[i].x, v[i].x, ss);
        ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss);
        ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    const size_t obase = (size_t)r * out_stride;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int j = i * THREADS + threadIdx.x;
        if (j >= n4) continue;
        const int c = j * 4;
        const float o0 = v[i].x * scale * wv[i].x;
        const float o1 = v[i].y * scale * wv[i].y;
        const float o2 = v[i].z * scale * wv[i].z;
        const float o3 = v[i].w * scale * wv[i].w;
        if (out_dtype == BFI_F32) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + obase + c) = make_float4(o0, o1, o2, o3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + obase + c) = packed;
        }
    }
}

extern "C" int bfi_rmsnorm(const void* x, int x_dtype, long x_stride, const int* rows, const void* w,
                           int w_dtype, void* out, int out_dtype, long out_stride, int n_rows, int width,
                           float eps, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(x_dtype) && dtype_ok(w_dtype) && dtype_ok(out_dtype), "rmsnorm: unknown dtype code");
    BFI_REQUIRE(n_rows >= 0 && width > 0, "rmsnorm: bad sizes rows=%d width=%d", n_rows, width);
    BFI_REQUIRE(x_stride >= width && out_stride >= width, "rmsnorm: row stride shorter than the row");
    if (n_rows == 0) return 0;
    const bool vec = x_dtype == BFI_F32 && width % 4 == 0 && x_stride % 4 == 0 && out_stride % 4 == 0 &&
                     ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0 && width <= 4 * 4 * 256;
    if (vec) {
#define BFI_NORM(V, T)                                                                                             \
    bfi_launch(rmsnorm_regs_kernel<V, T>, dim3(n_rows), dim3(T), 0, stream, (const float*)x, x_stride, rows, w,    \
               w_dtype, out, out_dtype, out_stride, width, eps)
        const bool many = n_rows > 4 * bfi_sm_count() && width <= 4 * 8 * 128;
        if (many) {
            const int vpt = (width / 4 + 127) / 128;
            if (vpt <= 1) BFI_NORM(1, 128);
            else if (vpt == 2) BFI_NORM(2, 128);
            else if (vpt <= 4) BFI_NORM(4, 128);
            else if (vpt <= 6) BFI_NORM(6, 128);
            else BFI_NORM(8, 128);
        } else {
            const int vpt = (width / 4 + 255) / 256;
            if (vpt <= 1) BFI_NORM(1, 256);
            else if (vpt == 2) BFI_NORM(2, 256);
            else if (vpt == 3) BFI_NORM(3, 256);
            else BFI_NORM(4, 256);
        }
#undef BFI_NORM
        return bfi_check_launch("rmsnorm");
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (x_dtype == BFI_F32)
        bfi_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, (const float*)x, x_stride, rows, w, w_dtype, out,
                                                              out_dtype, out_stride, width, eps);
    else
        bfi_launch(rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, (const bf16*)x, x_stride, rows, w, w_dtype, out,
                                                             out_dtype, out_stride, width, eps);
    return bfi_check_launch("rmsnorm");
}

// ------------------------------------------------------------------------------------------
// SiLU(gate) * up.  `interleaved` != 0: the input row holds gate_j, up_j at columns 2j, 2j+1;
// otherwise gate fills the first half of the row and up the second.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float silu_f32(float g) {
    // overflow-safe two-branch sigmoid, as the reference evaluates it
    float s;
    if (g >= 0.0f) {
        s = 1.0f / (1.0f + expf(-g));
    } else {
        const float z = expf(g);
        s = z / (1.0f + z);
    }
    return g * s;
}

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, long in_stride, T* __restrict__ out, long out_stride,
                                int n_rows, int inter, int interleaved) {
    pdl_trigger();
    pdl_wait();
    const long total = (long)n_rows * inter;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long r = i / inter;
        const int j = (int)(i - r * inter);
        const T* row = gu + r * in_stride;
        const float g = to_f32(interleaved ? row[2 * j] : row[j]);
        const float u = to_f32(interleaved ? row[2 * j + 1] : row[inter + j]);
        out[r * out_stride + j] = from_f32<T>(silu_f32(g) * u);
    }
}

extern "C" int bfi_silu_mul(const void* gu, long in_stride, void* out, long out_stride, int dtype, int n_rows,
                            int inter, int interleaved, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "silu_mul: unknown dtype code %d", dtype);
    BFI_REQUIRE(n_rows >= 0 && inter > 0, "silu_mul: bad sizes rows=%d width=%d", n_rows, inter);
    BFI_REQUIRE(in_stride >= 2L * inter && out_stride >= inter, "silu_mul: row stride shorter than the row");
    if (n_rows == 0) return 0;
    const long total = (long)n_rows * inter;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < bfi_sm_count() * 16L ? (total + threads - 1) / threads : bfi_sm_count() * 16L);
    if (dtype == BFI_F32)
        bfi_launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gu, in_stride, (float*)out, out_stride,
                                                               n_rows, inter, interleaved);
    else
        bfi_launch(silu_mul_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, (const bf16*)gu, in_stride, (bf16*)out, out_stride,
                                                              n_rows, inter, interleaved);
    return bfi_check_launch("silu_mul");
}

// ------------------------------------------------------------------------------------------
// After the QKV projection: per token and head, RMS norm over head_dim (q and k), rotate-half
// rotation by the token's position (q and k), then q back in place and k, v into the cache page
// of the token's slot.  One warp per (token, head); the head passes through shared memory so
// any head_dim that is a multiple of 16 (up to 512) works.
//
//   qkv          [tokens, (n_q + n_kv_in*2) * d]   n_kv_in = 0 when the run reads another run's cache
//   rope_table   [positions, rot_dim/2] of (cos, sin), float32, or null for no rotation
//   flags        bit 0: write k, v into the cache;  bit 1: write k back in place as well
// ------------------------------------------------------------------------------------------
#define QKR_WARPS 4
#define QKR_MAX_D 512

template <typename T>
__global__ void qk_norm_rope_cache_kernel(T* __restrict__ qkv, long token_stride, int n_tokens, int n_q, int n_kv,
                                          int d, const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w,
                                          int norm_dtype, float eps, const float2* __restrict__ rope_table,
                                          int rot_dim, int table_positions, const int* __restrict__ token_pos,
                                          const int* __restrict__ token_slot, T* __restrict__ k_pages,
                                          T* __restrict__ v_pages, const int* __restrict__ block_table,
                                          int table_stride, int flags, int* status) {
    pdl_trigger();
    pdl_wait();
    __shared__ float buf[QKR_WARPS][QKR_MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = n_q + 2 * n_kv;
    const long item = (long)blockIdx.x * QKR_WARPS + warp;
    if (item >= (long)n_tokens * heads) return;
    const int t = (int)(item / heads);
    const int hh = (int)(item - (long)t * heads);
    const int slot = token_slot[t];
    if (slot < 0) return;  // padding row
    const int pos = token_pos[t];
    const int kind = hh < n_q ? 0 : (hh < n_q + n_kv ? 1 : 2);  // q, k, v
    T* src = qkv + (size_t)t * token_stride + (size_t)hh * d;
    float* b = buf[warp];

    float ss = 0.0f;
    for (int j = lane; j < d; j += 32) {
        const float v = to_f32(src[j]);
        b[j] = v;
        ss = fmaf(v, v, ss);
    }
    const void* nw = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
    if (nw != nullptr) {
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)d + eps);
        for (int j = lane; j < d; j += 32) b[j] = b[j] * scale * load_as_f32(nw, norm_dtype, j);
    }
    __syncwarp();

    // destination
    T* dst_cache = nullptr;
    if (kind != 0 && (flags & 1)) {
        const int page = block_table[(size_t)slot * table_stride + pos / BFI_PAGE_TOKENS];
        if (page < 0) {
            if (lane == 0 && status) atomicOr(status, BFI_STATUS_NO_PAGE);
        } else {
            T* pages = kind == 1 ? k_pages : v_pages;
            const int h = kind == 1 ? hh - n_q : hh - n_q - n_kv;
            dst_cache = pages + (((size_t)page * n_kv + h) * BFI_PAGE_TOKENS + (pos % BFI_PAGE_TOKENS)) * d;
        }
    }
    const bool in_place = kind == 0 || (kind == 1 && (flags & 2));

    if (kind != 2 && rope_table != nullptr) {
        if (pos < 0 || pos >= table_positions) {
            if (lane == 0 && status) atomicOr(status, BFI_STATUS_BAD_POSITION);
            return;
        }
        const int half = rot_dim >> 1;
        const float2* cs = rope_table + (size_t)pos * half;
        for (int i = lane; i < half; i += 32) {
            const float2 c = cs[i];
            const float x0 = b[i], x1 = b[i + half];
            const float o0 = x0 * c.x - x1 * c.y;
            const float o1 = x0 * c.y + x1 * c.x;
            if (in_place) {
                src[i] = from_f32<T>(o0);
                src[i + half] = from_f32<T>(o1);
            }
            if (dst_cache) {
                dst_cache[i] = from_f32<T>(o0);
                dst_cache[i + half] = from_f32<T>(o1);
            }
        }
        for (int j = rot_dim + lane; j < d; j += 32) {
            if (in_place) src[j] = from_f32<T>(b[j]);
            if (dst_cache) dst_cache[j] = from_f32<T>(b[j]);
        }
    } else {
        for (int j = lane; j < d; j += 32) {
            if (in_place && nw != nullptr) src[j] = from_f32<T>(b[j]);
            if (dst_cache) dst_cache[j] = from_f32<T>(b[j]);
        }
    }
}

// The same for bfloat16 heads of 64 or 128 values with the rotation over the whole head: a lane
// owns 4 consecutive values of the head's first half and the 4 values half a head further on, which
// are their rotation partners (two 8-byte accesses per head), so the rotation needs no other lane
// and nothing goes through shared memory.  LANES = head_dim / 8 lanes per head; a warp handles
// QKV_UNROLL * 32 / LANES consecutive heads of one token, whose position, page and rotation
// factors it fetches once.
// QKV_UNROLL: heads a lane group handles, their loads in flight together (1 for few tokens, where
// more warps matter more)
template <int D, int QKV_UNROLL>
__global__ void __launch_bounds__(128)
qk_norm_rope_cache_vec_kernel(bf16* __restrict__ qkv, long token_stride, int n_tokens, int n_q, int n_kv,
                              const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int norm_dtype,
                              float eps, const float2* __restrict__ rope_table, int table_positions,
                              const int* __restrict__ token_pos, const int* __restrict__ token_slot,
                              bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, const int* __restrict__ block_table,
                              int table_stride, int flags, int* status) {
    pdl_trigger();
    constexpr int LANES = D / 8;                        // a lane owns 4 + 4 values
    constexpr int HALF = D / 2;
    constexpr int PER_WARP = 32 / LANES;
    constexpr int HPW = PER_WARP * QKV_UNROLL;          // consecutive heads of one token per warp
    const int lane = threadIdx.x & 31, sub = lane % LANES;
    const int heads = n_q + 2 * n_kv;
    const int groups = (heads + HPW - 1) / HPW;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)n_tokens * groups) return;
    const int t = (int)(item / groups);
    const int head_base = (int)(item - (long)t * groups) * HPW + lane / LANES;
    bf16* row = qkv + (size_t)t * token_stride + sub * 4;

    const int slot = token_slot[t];
    const int pos = token_pos[t];
    if (slot < 0) return;
    const bool has_rope = rope_table != nullptr;
    const bool bad_pos = has_rope && (pos < 0 || pos >= table_positions);
    // rotation factors of this lane's 4 pairs and the norm weights of its 8 values, as vector loads
    float2 cs[4];
    float wq[8], wk[8];                                 // [0..3] first half, [4..7] second half
    if (has_rope && !bad_pos) {
        const float4* src = reinterpret_cast<const float4*>(rope_table + (size_t)pos * HALF + sub * 4);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float4 t4 = src[j];
            cs[2 * j] = make_float2(t4.x, t4.y);
            cs[2 * j + 1] = make_float2(t4.z, t4.w);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) cs[j] = make_float2(1.0f, 0.0f);
    }
    auto unpack4 = [](uint2 raw, float* dst) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        dst[0] = __low2float(a), dst[1] = __high2float(a), dst[2] = __low2float(b), dst[3] = __high2float(b);
    };
    auto load_w8 = [&](const void* w, float (&dst)[8]) {
        if (w == nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = 1.0f;
        } else if (norm_dtype == BFI_BF16 && ((uintptr_t)w & 7) == 0) {
            const bf16* wb = reinterpret_cast<const bf16*>(w) + sub * 4;
            unpack4(*reinterpret_cast<const uint2*>(wb), dst);
            unpack4(*reinterpret_cast<const uint2*>(wb + HALF), dst + 4);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                dst[j] = load_as_f32(w, norm_dtype, sub * 4 + j);
                dst[4 + j] = load_as_f32(w, norm_dtype, HALF + sub * 4 + j);
            }
        }
    };
    load_w8(q_norm_w, wq);
    load_w8(k_norm_w, wk);
    int page = 0;
    if (flags & 1) page = block_table[(size_t)slot * table_stride + pos / BFI_PAGE_TOKENS];
    // the token's slot, position, page, rotation factors and the norm weights were all there before this
    // step's kernels began; only the heads themselves come from the kernel before this one
    pdl_wait();
    uint2 raw_lo[QKV_UNROLL], raw_hi[QKV_UNROLL];
#pragma unroll
    for (int u = 0; u < QKV_UNROLL; ++u) {
        const int hh = head_base + u * PER_WARP;
        const bool live = hh < heads;
        raw_lo[u] = live ? *reinterpret_cast<const uint2*>(row + (size_t)hh * D) : make_uint2(0u, 0u);
        raw_hi[u] = live ? *reinterpret_cast<const uint2*>(row + (size_t)hh * D + HALF) : make_uint2(0u, 0u);
    }
    if (bad_pos) {
        if (lane == 0 && status) atomicOr(status, BFI_STATUS_BAD_POSITION);
        return;
    }
    if ((flags & 1) && page < 0 && lane == 0 && status && head_base + (QKV_UNROLL - 1) * PER_WARP >= n_q)
        atomicOr(status, BFI_STATUS_NO_PAGE);

#pragma unroll
    for (int u = 0; u < QKV_UNROLL; ++u) {
        const int hh = head_base + u * PER_WARP;
        const bool live = hh < heads;
        const int kind = hh < n_q ? 0 : (hh < n_q + n_kv ? 1 : 2);
        uint2 out_lo = raw_lo[u], out_hi = raw_hi[u];
        const bool normed = kind == 0 ? q_norm_w != nullptr : (kind == 1 && k_norm_w != nullptr);
        const bool rotate = kind != 2 && has_rope;
        // a warp's lane groups may hold heads of different kinds: the shuffles are run by all lanes
        // or by none (value heads, which are only copied, mostly fill warps of their own)
        float v[8];
        float ss = 0.0f;
        if (__any_sync(0xffffffffu, normed || rotate)) {
            unpack4(raw_lo[u], v);
            unpack4(raw_hi[u], v + 4);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        }
        if (normed || rotate) {
            if (normed) {
                const float scale = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = v[j] * scale * (kind == 0 ? wq[j] : wk[j]);
            }
            float o8[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o8[j] = rotate ? v[j] * cs[j].x - v[4 + j] * cs[j].y : v[j];
                o8[4 + j] = rotate ? v[4 + j] * cs[j].x + v[j] * cs[j].y : v[4 + j];
            }
            __nv_bfloat162 p0 = __floats2bfloat162_rn(o8[0], o8[1]), p1 = __floats2bfloat162_rn(o8[2], o8[3]);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(o8[4], o8[5]), p3 = __floats2bfloat162_rn(o8[6], o8[7]);
            out_lo = make_uint2(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1));
            out_hi = make_uint2(*reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
        }
        if (!live) continue;
        const bool in_place = kind == 0 || (kind == 1 && (flags & 2));
        if (in_place && (normed || rotate)) {
            *reinterpret_cast<uint2*>(row + (size_t)hh * D) = out_lo;
            *reinterpret_cast<uint2*>(row + (size_t)hh * D + HALF) = out_hi;
        }
        if (kind != 0 && (flags & 1) && page >= 0) {
            bf16* pages = kind == 1 ? k_pages : v_pages;
            const int h = kind == 1 ? hh - n_q : hh - n_q - n_kv;
            bf16* dst = pages + (((size_t)page * n_kv + h) * BFI_PAGE_TOKENS + (pos % BFI_PAGE_TOKENS)) * D + sub * 4;
            *reinterpret_cast<uint2*>(dst) = out_lo;
            *reinterpret_cast<uint2*>(dst + HALF) = out_hi;
        }
    }
}

extern "C" int bfi_qk_norm_rope_cache(void* qkv, int dtype, long token_stride, int n_tokens, int n_q, int n_kv,
                                      int d, const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps,
                                      const void* rope_table, int rot_dim, int table_positions,
                                      const int* token_pos, const int* token_slot, void* k_pages, void* v_pages,
                                      const int* block_table, int table_stride, int flags, int* status,
                                      cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype) && dtype_ok(norm_dtype), "qk_norm_rope_cache: unknown dtype code");
    BFI_REQUIRE(n_tokens >= 0 && n_q >= 0 && n_kv >= 0 && n_q + n_kv > 0, "qk_norm_rope_cache: bad head counts q=%d kv=%d",
                n_q, n_kv);
    BFI_REQUIRE(d > 0 && d % 2 == 0 && d <= QKR_MAX_D, "qk_norm_rope_cache: head_dim %d must be even and at most %d",
                d, QKR_MAX_D);
    BFI_REQUIRE(token_stride >= (long)(n_q + 2 * n_kv) * d, "qk_norm_rope_cache: token stride shorter than the heads");
    if (rope_table) {
        BFI_REQUIRE(rot_dim > 0 && rot_dim % 2 == 0 && rot_dim <= d,
                    "qk_norm_rope_cache: rotary width %d must be even and at most head_dim %d", rot_dim, d);
        BFI_REQUIRE(table_positions > 0, "qk_norm_rope_cache: empty rotation table");
    }
    if ((flags & 1) && n_kv > 0)
        BFI_REQUIRE(k_pages && v_pages && block_table && table_stride > 0, "qk_norm_rope_cache: cache write without a cache");
    if (n_tokens == 0) return 0;
    const long items = (long)n_tokens * (n_q + 2 * n_kv);
    // bfloat16 heads of 64 or 128 rotated over the whole head (or not at all): the vector kernel
    const bool vec = dtype == BFI_BF16 && (d == 64 || d == 128) && (rope_table == nullptr || rot_dim == d) &&
                     token_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0;
    if (vec) {
        const int unroll = n_tokens >= 512 ? 4 : 1;      // many tokens: more bytes in flight per warp; few: more warps
        const int heads_per_warp = (32 / (d / 8)) * unroll;
        const long warps = (long)n_tokens * ((n_q + 2 * n_kv + heads_per_warp - 1) / heads_per_warp);
        const int vblocks = (int)((warps + 3) / 4);
#define BFI_QKV_VEC(DD, UU)                                                                                               \
    bfi_launch(qk_norm_rope_cache_vec_kernel<DD, UU>, dim3(vblocks), dim3(128), 0, stream, (bf16*)qkv, token_stride,      \
               n_tokens, n_q, n_kv, q_norm_w, k_norm_w, norm_dtype, eps, (const float2*)rope_table, table_positions,       \
               token_pos, token_slot, (bf16*)k_pages, (bf16*)v_pages, block_table, table_stride, flags, status)
        if (d == 128) {
            if (unroll == 1) BFI_QKV_VEC(128, 1);
            else BFI_QKV_VEC(128, 4);
        } else {
            if (unroll == 1) BFI_QKV_VEC(64, 1);
            else BFI_QKV_VEC(64, 4);
        }
#undef BFI_QKV_VEC
        return bfi_check_launch("qk_norm_rope_cache_vec");
    }
    const int blocks = (int)((items + QKR_WARPS - 1) / QKR_WARPS);
    if (dtype == BFI_F32)
        bfi_launch(qk_norm_rope_cache_kernel<float>, dim3(blocks), dim3(QKR_WARPS * 32), 0, stream, 
            (float*)qkv, token_stride, n_tokens, n_q, n_kv, d, q_norm_w, k_norm_w, norm_dtype, eps,
            (const float2*)rope_table, rot_dim, table_positions, token_pos, token_slot, (float*)k_pages,
            (float*)v_pages, block_table, table_stride, flags, status);
    else
        bfi_launch(qk_norm_rope_cache_kernel<bf16>, dim3(blocks), dim3(QKR_WARPS * 32), 0, stream, 
            (bf16*)qkv, token_stride, n_tokens, n_q, n_kv, d, q_norm_w, k_norm_w, norm_dtype, eps,
            (const float2*)rope_table, rot_dim, table_positions, token_pos, token_slot, (bf16*)k_pages,
            (bf16*)v_pages, block_table, table_stride, flags, status);
    return bfi_check_launch("qk_norm_rope_cache");
}

// ------------------------------------------------------------------------------------------
// Small utilities
// ------------------------------------------------------------------------------------------
// out[i] += add[i]  (float32 residual stream += an activation)
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ y, long n) {
    pdl_trigger();
    pdl_wait();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        x[i] += to_f32(y[i]);
}

extern "C" int bfi_residual_add(float* x, const void* y, int y_dtype, long n, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(y_dtype), "residual_add: unknown dtype code %d", y_dtype);
    if (n <= 0) return 0;
    const int threads = 256;
    const long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < bfi_sm_count() * 16L ? want : bfi_sm_count() * 16L);
    if (y_dtype == BFI_F32)
        bfi_launch(residual_add_kernel<float>, dim3(blocks), dim3(threads), 0, stream, x, (const float*)y, n);
    else
        bfi_launch(residual_add_kernel<bf16>, dim3(blocks), dim3(threads), 0, stream, x, (const bf16*)y, n);
    return bfi_check_launch("residual_add");
}

BFI_TRACE_EXPORT(elementwise)
