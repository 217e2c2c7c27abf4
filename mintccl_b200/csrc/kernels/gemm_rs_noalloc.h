// Allocation-free entry point for the single-rank GEMM -> reduce-scatter kernel.
//
// This entry point has no counterpart in the reference library; it exists for hosts that must not
// allocate device memory once they are running: code inside a latency-critical serving loop, a plugin
// loaded into a process whose memory pool is owned by somebody else, or a caller that has handed all
// device memory to its own allocator and would make cudaMalloc fail or stall.  The regular entry point
// (mt_gemm_rs) keeps its partial tiles and arrival counters in the communicator's heap, which is
// allocated when the communicator is created.  This variant keeps them in a fixed array that is part of
// the library image, so it needs no communicator and calls no allocating routine.
#pragma once
#include <stdint.h>
#include "../device/layout.h"

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch can hold: M <= 2048 rows and N <= 2048 columns of bf16 partial
// tiles (8 MiB) plus counters and a descriptor; about 8.1 MiB of device memory on every GPU that loads
// the library, held until the process exits.
#define MT_NOALLOC_MAX_M 2048
#define MT_NOALLOC_MAX_N 2048

// out[M, N] = A[M, K] * B[N, K]^T (bf16 in, fp32 accumulate, bf16 out) computed by the GEMM ->
// reduce-scatter kernel on one rank, with its scratch in the library's built-in array.
//
//  * M must be a multiple of 128, N of 256, K of 64; M <= MT_NOALLOC_MAX_M and N <= MT_NOALLOC_MAX_N,
//    otherwise the call fails with -1 and mt_last_error() says which limit was exceeded.
//  * A, B, out are device pointers on the current device, 16-byte aligned.
//  * The first call on each device looks up the device address of the scratch array and writes a small
//    descriptor into it (one synchronous copy).  Make that first call before starting a stream capture.
//  * All calls on a device share the one scratch array, which keeps the previous call's contents; the
//    counters are cleared on the caller's stream before every launch.  Two calls that overlap on the GPU
//    (different streams, no dependency) race on it: serialise them.
//  * Calls no cudaMalloc / cudaFree and no allocating library routine.
// Returns 0 on success, -1 on error.
int mt_gemm_rs_single_noalloc(void* stream, const void* A, const void* B, void* out, int M, int N, int K);

// The kernel's waits are bounded: one that runs out of time records {code, where, expected, seen} and raises
// `abort` in a status record that lives in the same built-in array (the call itself has long returned 0, and
// `out` is then incomplete).  This copies the record of the current device to `*out` after synchronising the
// device, and zeroes it when `clear` is non-zero; code == 0 and abort == 0 mean every call so far completed.
// Allocates nothing.  Returns 0 on success, -1 on error.
int mt_gemm_rs_single_noalloc_status(MtStatus* out, int clear);

#ifdef __cplusplus
}
#endif
