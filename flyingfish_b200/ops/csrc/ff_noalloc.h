// Allocation-free entry point of the kernel library. It has no counterpart in the reference
// engine, whose host runtime always owns an allocator.
//
// ff_gemm_skinny_noalloc computes Y[M,N] = X[M,K] * W[N,K]^T (BF16 in, FP32 accumulate, BF16 out)
// for decode-sized M (1..128) exactly like ff_gemm_skinny, but takes no scratch from the caller:
// the split-K partial sums and tile counters live in a fixed array inside the library. It is
// meant for callers that cannot allocate device memory when they need the product -- a host
// whose allocator is frozen after start-up, a plugin with a fixed memory budget, or a C caller
// that only owns its inputs and outputs.
//
// Rules for the caller:
//   * X, W, Y are device pointers owned by the caller; ldx/ldw/ldy are row pitches in elements
//     (multiples of 8); `status` may be null or point to int32[4] in device memory.
//   * The partial-sum slots (the scratch size ff_gemm_skinny_plan(M, N, K) reports: 2 * grid * M * 128 * 4
//     bytes for problems it runs as stream-K over 128-row weight tiles with grid <= 148 CTAs, none
//     for cluster split-K) must fit in FF_NOALLOC_SCRATCH_BYTES and the weight tiles in
//     FF_NOALLOC_MAX_TILES; otherwise, and for M > 128, the call returns -5 and launches nothing.
//     For a layer wide enough to occupy all 148 CTAs the limit is reached above M = 55 tokens.
//   * The first call on each device looks up the array's device address; issue it before any
//     stream capture begins on that device, with the device that owns `stream` current.
//   * All calls share the array, so calls that can overlap on the GPU race; order them on one
//     stream (or with events).
//   * Returns 0, a negative host-side refusal code, or a positive cudaError_t.
#pragma once
#include <cuda_runtime.h>

#define FF_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)
#define FF_NOALLOC_MAX_TILES 2048

extern "C" int ff_gemm_skinny_noalloc(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                                      int ldy, int* status, cudaStream_t stream);
