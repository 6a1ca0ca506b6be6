// Matrix products on the CUDA cores, float32 multiply-add, for every combination of storage
// types and every size: C[M,N] = A[M,K] * W[N,K]^T with W stored [out, in] row-major as the
// reference stores it (crates/bfi-core/src/cpu.rs:78-90, 498-514).
//
// These kernels are the whole of the true 32-bit path (no tensor-core mode is involved) and the
// fallback of the bfloat16 path for shapes and dtype pairs the tensor-core kernels refuse.
//
// Epilogues:
//   0  C = acc                         (C in c_dtype)
//   1  C += acc                        (C float32: the residual stream)
//   2  C[m, j] = silu(acc[m,2j]) * acc[m,2j+1]   (W rows interleaved gate/up; C has N/2 columns)
#include "common.cuh"

#define EPI_STORE 0
#define EPI_ACCUMULATE 1
#define EPI_SWIGLU 2

__device__ __forceinline__ float silu_mul_f32(float g, float u) {
    float s;
    if (g >= 0.0f) {
        s = 1.0f / (1.0f + expf(-g));
    } else {
        const float z = expf(g);
        s = z / (1.0f + z);
    }
    return g * s * u;
}

// ------------------------------------------------------------------------------------------
// Tiled kernel: 64x64 output tile, K step 16, 256 threads, 4x4 outputs per thread.
// ------------------------------------------------------------------------------------------
#define TM 64
#define TN 64
#define TK 16
#define TPAD 4

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
gemm_tile_kernel(const TA* __restrict__ A, long lda, const TW* __restrict__ W, long ldw, void* __restrict__ C,
                 int c_dtype, long ldc, int M, int N, int K, int epilogue) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float As[TK][TM + TPAD];
    __shared__ __align__(16) float Ws[TK][TN + TPAD];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int ty = tid >> 4, tx = tid & 15;
    // loader mapping: 4 consecutive k of one row
    const int lrow = tid >> 2, lk = (tid & 3) * 4;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        {
            const int gm = m0 + lrow;
            const TA* ap = A + (size_t)gm * lda + k0 + lk;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const int gk = k0 + lk + kk;
                As[lk + kk][lrow] = (gm < M && gk < K) ? to_f32(ap[kk]) : 0.0f;
            }
            const int gn = n0 + lrow;
            const TW* wp = W + (size_t)gn * ldw + k0 + lk;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const int gk = k0 + lk + kk;
                Ws[lk + kk][lrow] = (gn < N && gk < K) ? to_f32(wp[kk]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w};
            const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
        if (epilogue == EPI_SWIGLU) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int gn = n0 + tx * 4 + j;
                if (gn + 1 < N)
                    store_from_f32(C, c_dtype, (size_t)gm * ldc + (gn >> 1), silu_mul_f32(acc[i][j], acc[i][j + 1]));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gn = n0 + tx * 4 + j;
                if (gn >= N) continue;
                const size_t idx = (size_t)gm * ldc + gn;
                if (epilogue == EPI_ACCUMULATE)
                    reinterpret_cast<float*>(C)[idx] += acc[i][j];
                else
                    store_from_f32(C, c_dtype, idx, acc[i][j]);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Few rows (M <= 8 per pass): one warp per pair of W rows, lanes stride over K, so each weight
// is read once for all rows of the pass.  Used for decode steps of the 32-bit path and as the
// bfloat16 fallback.
// ------------------------------------------------------------------------------------------
template <typename TA, typename TW, int MB>
__global__ void __launch_bounds__(256)
gemv_rows_kernel(const TA* __restrict__ A, long lda, const TW* __restrict__ W, long ldw, void* __restrict__ C,
                 int c_dtype, long ldc, int m_base, int M, int N, int K, int epilogue) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + warp;
    const int n_a = pair * 2, n_b = n_a + 1;
    if (n_a >= N) return;
    const bool has_b = n_b < N;
    const TW* wa = W + (size_t)n_a * ldw;
    const TW* wb = W + (size_t)(has_b ? n_b : n_a) * ldw;
    float acc_a[MB], acc_b[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc_a[m] = acc_b[m] = 0.0f;
    for (int k = lane; k < K; k += 32) {
        const float va = to_f32(wa[k]);
        const float vb = to_f32(wb[k]);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const int gm = m_base + m;
            const float x = gm < M ? to_f32(A[(size_t)gm * lda + k]) : 0.0f;
            acc_a[m] = fmaf(va, x, acc_a[m]);
            acc_b[m] = fmaf(vb, x, acc_b[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < MB; ++m) {
        acc_a[m] = warp_sum(acc_a[m]);
        acc_b[m] = warp_sum(acc_b[m]);
    }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const int gm = m_base + m;
            if (gm >= M) continue;
            if (epilogue == EPI_SWIGLU) {
                if (has_b) store_from_f32(C, c_dtype, (size_t)gm * ldc + (n_a >> 1), silu_mul_f32(acc_a[m], acc_b[m]));
            } else if (epilogue == EPI_ACCUMULATE) {
                reinterpret_cast<float*>(C)[(size_t)gm * ldc + n_a] += acc_a[m];
                if (has_b) reinterpret_cast<float*>(C)[(size_t)gm * ldc + n_b] += acc_b[m];
            } else {
                store_from_f32(C, c_dtype, (size_t)gm * ldc + n_a, acc_a[m]);
                if (has_b) store_from_f32(C, c_dtype, (size_t)gm * ldc + n_b, acc_b[m]);
            }
        }
    }
}

template <typename TA, typename TW>
static int launch_simt(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype, long ldc, int M, int N,
                       int K, int epilogue, cudaStream_t stream) {
    if (M <= 16) {
        const int warps = 8;
        const int pairs = (N + 1) / 2;
        const int blocks = (pairs + warps - 1) / warps;
        for (int m_base = 0; m_base < M; m_base += 8) {
            const int left = M - m_base;
            if (left >= 5)
                bfi_launch(gemv_rows_kernel<TA, TW, 8>, dim3(blocks), dim3(warps * 32), 0, stream, (const TA*)A, lda, (const TW*)W, ldw, C,
                                                                              c_dtype, ldc, m_base, M, N, K, epilogue);
            else if (left >= 3)
                bfi_launch(gemv_rows_kernel<TA, TW, 4>, dim3(blocks), dim3(warps * 32), 0, stream, (const TA*)A, lda, (const TW*)W, ldw, C,
                                                                              c_dtype, ldc, m_base, M, N, K, epilogue);
            else if (left == 2)
                bfi_launch(gemv_rows_kernel<TA, TW, 2>, dim3(blocks), dim3(warps * 32), 0, stream, (const TA*)A, lda, (const TW*)W, ldw, C,
                                                                              c_dtype, ldc, m_base, M, N, K, epilogue);
            else
                bfi_launch(gemv_rows_kernel<TA, TW, 1>, dim3(blocks), dim3(warps * 32), 0, stream, (const TA*)A, lda, (const TW*)W, ldw, C,
                                                                              c_dtype, ldc, m_base, M, N, K, epilogue);
        }
        return bfi_check_launch("gemv_rows");
    }
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    BFI_REQUIRE(grid.y <= 65535, "gemm_simt: M=%d is too large for one launch", M);
    bfi_launch(gemm_tile_kernel<TA, TW>, dim3(grid), dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, ldw, C, c_dtype, ldc, M, N, K,
                                                      epilogue);
    return bfi_check_launch("gemm_tile");
}

extern "C" int bfi_gemm_simt(const void* A, int a_dtype, long lda, const void* W, int w_dtype, long ldw, void* C,
                             int c_dtype, long ldc, int M, int N, int K, int epilogue, cudaStream_t stream) {
    BFI_REQUIRE(dtype_ok(a_dtype) && dtype_ok(w_dtype) && dtype_ok(c_dtype), "gemm_simt: unknown dtype code");
    BFI_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
    BFI_REQUIRE(lda >= K && ldw >= K, "gemm_simt: a row stride is shorter than K=%d", K);
    BFI_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_simt: unknown epilogue %d", epilogue);
    if (epilogue == EPI_ACCUMULATE) BFI_REQUIRE(c_dtype == BFI_F32, "gemm_simt: accumulation needs a float32 output");
    if (epilogue == EPI_SWIGLU) {
        BFI_REQUIRE(N % 2 == 0, "gemm_simt: the gated epilogue needs an even N, got %d", N);
        BFI_REQUIRE(ldc >= N / 2, "gemm_simt: output row stride shorter than N/2");
    } else {
        BFI_REQUIRE(ldc >= N, "gemm_simt: output row stride shorter than N=%d", N);
    }
    if (M == 0) return 0;
    // chunk M so that gridDim.y stays legal
    const int max_rows = 65535 * TM;
    for (int m0 = 0; m0 < M; m0 += max_rows) {
        const int rows = M - m0 < max_rows ? M - m0 : max_rows;
        const char* a = (const char*)A + (size_t)m0 * lda * dtype_size(a_dtype);
        const size_t c_cols_stride = (size_t)m0 * ldc * dtype_size(c_dtype);
        char* c = (char*)C + c_cols_stride;
        int rc;
        if (a_dtype == BFI_F32 && w_dtype == BFI_F32)
            rc = launch_simt<float, float>(a, lda, W, ldw, c, c_dtype, ldc, rows, N, K, epilogue, stream);
        else if (a_dtype == BFI_F32 && w_dtype == BFI_BF16)
            rc = launch_simt<float, bf16>(a, lda, W, ldw, c, c_dtype, ldc, rows, N, K, epilogue, stream);
        else if (a_dtype == BFI_BF16 && w_dtype == BFI_F32)
            rc = launch_simt<bf16, float>(a, lda, W, ldw, c, c_dtype, ldc, rows, N, K, epilogue, stream);
        else
            rc = launch_simt<bf16, bf16>(a, lda, W, ldw, c, c_dtype, ldc, rows, N, K, epilogue, stream);
        if (rc) return rc;
    }
    return 0;
}

BFI_TRACE_EXPORT(gemm_simt)
