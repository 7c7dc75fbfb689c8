// Allocation-free entry point of the dense tensor-core GEMM.
//
// This entry point has no counterpart in the reference implementation; it exists for embedders of
// this library that are not allowed to allocate device memory at call time:
//   * hosts that hand every library a fixed device-memory budget up front and treat any later
//     cudaMalloc as a fault (plugin hosts, co-located services with hard per-tenant limits);
//   * callers on a latency-critical path where cudaMalloc / cudaFree would serialise the whole
//     device behind an implicit synchronisation;
//   * callers whose device heap is owned by another allocator that they do not want to re-enter
//     from inside a kernel library.
// The regular entry point (mlcb_gemm) expects the caller to provide split-K scratch; here the
// scratch is a fixed array inside the library image instead.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the split-K reduction may use through this entry point. The array lives in the
// library image, so every GPU that loads the library carries this much device memory until the
// process exits, whether or not the entry point is ever called.
#define MLCB_NOALLOC_SCRATCH_BYTES (8u << 20)
// Largest number of output tiles (ceil(M / tokens-per-tile) * ceil(N / 128)) whose arrival counters
// fit in the built-in counter array.
#define MLCB_NOALLOC_MAX_TILES 1024

// Y[M, N] = X[M, K] . W[N, K]^T for 16-bit inputs (ab_fmt 0 = fp16, 1 = bf16), output in the same
// 16-bit type. x: row-major with leading dimension ldx, w: row-major [N, K], y: leading dimension
// ldy (all in elements). K and ldx must be multiples of 8, pointers 16-byte aligned.
//
// Performs no cudaMalloc / cudaFree and calls no allocating library routine. Split-K partial sums
// and tile counters live in a file-scope __device__ array of MLCB_NOALLOC_SCRATCH_BYTES (+ counters).
//
// * The first call on each device looks up the device address of that array (a one-time set-up,
//   done with that device current). Make that first call outside of any stream capture.
// * All calls on a device share the one array, and it keeps whatever the previous call left in it;
//   the entry point clears the tile counters itself before each launch. Two calls that can overlap
//   on the GPU (different streams, no ordering between them) race on the scratch: order them.
// * Shapes whose split-K scratch would exceed the built-in array, or with more tiles than
//   MLCB_NOALLOC_MAX_TILES, are rejected: the function returns MLCB_NOALLOC_TOO_LARGE and
//   mlcb_gemm_noalloc_last_error() describes the limit. Nothing is launched in that case.
//
// Returns 0 on success, a negative MLCB_NOALLOC_* code for rejected arguments, or a positive
// cudaError_t value if the runtime reported an error.
#define MLCB_NOALLOC_BAD_ARGUMENT (-1)
#define MLCB_NOALLOC_TOO_LARGE (-2)
#define MLCB_NOALLOC_NO_DRIVER_ENTRY (-4)
int mlcb_gemm_noalloc(const void* x, const void* w, void* y, int M, int N, int K, int ldx, int ldy,
                      int ab_fmt, int* status, cudaStream_t stream);

// Human-readable description of the last failure of mlcb_gemm_noalloc on the calling thread
// (empty string if the last call succeeded).
const char* mlcb_gemm_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
