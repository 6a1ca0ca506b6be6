// A matrix product for callers that may not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for hosts that cannot
// hand this library a scratch buffer of their own making: programs that gave all device memory to
// an arena at start-up and never call the CUDA allocator afterwards, plug-ins that run inside
// another runtime's callback where cudaMalloc (which may synchronise the whole device) is
// forbidden, and processes with a fixed, audited memory plan.  Such a caller still owns its inputs
// and outputs; only the kernel's private scratch is the library's problem.
//
//   C[M,N] = A[M,K] * W[N,K]^T,  bfloat16 x bfloat16, float32 accumulation, M <= 64,
//   epilogue 0 store / 1 add into float32 C / 2 SiLU(gate)*up over interleaved rows of W,
//
// exactly as bfi_skinny_gemm_bf16 computes it (same kernel, same fixed summation order).  When K
// is split between blocks the partial sums and the per-tile counters live in ONE array in the
// library's own device image:
//
//   static __device__ __align__(256) float bfi_static_scratch[BFI_STATIC_SCRATCH_FLOATS];   // 4 MiB
//
// Every GPU that loads the library holds these 4 MiB until the process exits.  A shape whose plan
// needs more (bfi_skinny_gemm_scratch tells how much) is refused with an error; nothing is
// launched.  The function calls no cudaMalloc, cudaFree or any other allocating routine.
//
// The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
// that device current) and remembers it; make that first call outside any stream capture.
//
// All calls share the array and find in it whatever the last call left: the counter region is
// cleared on the stream at the start of every call, and the partial sums are overwritten before
// they are read.  Two calls that overlap on the GPU (different streams, or different host threads
// on one device) would race on it: run them on one stream.
//
// Returns 0 on success, 1 on error (bfi_last_error() has the text), 2 when the shape is not one
// the kernel takes (K not a multiple of 8, unaligned rows, M > 64); nothing is launched for 1 or 2.
#pragma once

#include <cuda_runtime.h>

#define BFI_STATIC_SCRATCH_FLOATS (1 << 20)     // 4 MiB in all
#define BFI_STATIC_COUNTER_SLOTS (1 << 14)      // the first 64 KiB of it hold the per-tile counters

extern "C" int bfi_skinny_gemm_bf16_static(const void* A, long lda, const void* W, long ldw, void* C, int c_dtype,
                                           long ldc, int M, int N, int K, int epilogue, cudaStream_t stream);
