// Utility kernels beside the model's own: the seeded random fill of the random-weights mode and
// the conversion between the two storage types.
//
// The fill is a closed formula, value = f(key, element index), so that any implementation can
// rebuild a tensor bit for bit (the reference builds its toy models from a closed formula for the
// same reason: crates/bfi-models/src/lib.rs:52-79).  For element i of a tensor with 64-bit key k:
//
//     x_j = mix64(k + (2 i + j + 1) * 0x9E3779B97F4A7C15)        j = 0, 1     (wrapping)
//     s   = sum of the eight 16-bit fields of x_0 and x_1
//     c   = 2 s - 8 * 65535                                       an integer, |c| <= 524280
//     v   = offset + float(c) * scale                             one multiply, one add, float32
//
// mix64 is the splitmix64 finalizer.  s is a sum of eight uniform integers (Irwin-Hall), close to
// normal with standard deviation 65536 * sqrt(2/3); the host passes scale = std / (131072 *
// sqrt(2/3)) rounded to float32, so both sides multiply by the same number.  Every step is exact
// integer arithmetic or a single correctly rounded float32 operation, which is what makes the
// values the same on every machine.
#include "common.cuh"

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ int fields16(unsigned long long x) {
    return (int)(x & 0xFFFF) + (int)((x >> 16) & 0xFFFF) + (int)((x >> 32) & 0xFFFF) + (int)(x >> 48);
}

template <typename T>
__global__ void fill_random_kernel(T* __restrict__ out, long n, unsigned long long key, float scale, float offset) {
    pdl_trigger();
    pdl_wait();
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const unsigned long long base = key + (2ull * (unsigned long long)i + 1ull) * 0x9E3779B97F4A7C15ull;
        const int s = fields16(mix64(base)) + fields16(mix64(base + 0x9E3779B97F4A7C15ull));
        const float c = (float)(2 * s - 8 * 65535);
        out[i] = from_f32<T>(__fadd_rn(offset, __fmul_rn(c, scale)));
    }
}

template <typename S, typename D>
__global__ void convert_kernel(const S* __restrict__ src, D* __restrict__ dst, long n) {
    pdl_trigger();
    pdl_wait();
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = from_f32<D>(to_f32(src[i]));
}

static int grid_for(long n, int threads) {
    const long want = (n + threads - 1) / threads;
    const long cap = (long)bfi_sm_count() * 16;
    return (int)(want < cap ? want : cap);
}

// out[i] = offset + c_i * scale for i < n, c_i from the formula above; out is contiguous.
extern "C" int bfi_fill_random(void* out, int dtype, long n, unsigned long long key, float scale, float offset,
                               cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(dtype), "fill_random: unknown dtype code %d", dtype);
    if (n <= 0) return 0;
    const int threads = 256;
    if (dtype == BFI_F32)
        bfi_launch(fill_random_kernel<float>, dim3(grid_for(n, threads)), dim3(threads), 0, stream, (float*)out, n, key,
                   scale, offset);
    else
        bfi_launch(fill_random_kernel<bf16>, dim3(grid_for(n, threads)), dim3(threads), 0, stream, (bf16*)out, n, key,
                   scale, offset);
    return bfi_check_launch("fill_random");
}

// dst[i] = src[i] for i < n between float32 and bfloat16 (round to nearest even); both contiguous.
extern "C" int bfi_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long n, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(src_dtype) && dtype_ok(dst_dtype), "convert: unknown dtype code %d -> %d", src_dtype, dst_dtype);
    if (n <= 0) return 0;
    const int threads = 256;
    const dim3 grid(grid_for(n, threads)), block(threads);
    if (src_dtype == BFI_F32 && dst_dtype == BFI_BF16)
        bfi_launch(convert_kernel<float, bf16>, grid, block, 0, stream, (const float*)src, (bf16*)dst, n);
    else if (src_dtype == BFI_BF16 && dst_dtype == BFI_F32)
        bfi_launch(convert_kernel<bf16, float>, grid, block, 0, stream, (const bf16*)src, (float*)dst, n);
    else if (src_dtype == BFI_F32)
        bfi_launch(convert_kernel<float, float>, grid, block, 0, stream, (const float*)src, (float*)dst, n);
    else
        bfi_launch(convert_kernel<bf16, bf16>, grid, block, 0, stream, (const bf16*)src, (bf16*)dst, n);
    return bfi_check_launch("convert");
}
