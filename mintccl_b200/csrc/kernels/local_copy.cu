// Copy inside one GPU: what every collective of a one-rank communicator amounts to (the contribution of the only
// rank is the result).  The ring kernels handle that case too, but they are built around FIFO steps (one
// 512-thread CTA per SM, a block barrier per step) and reach 0.6 of the copy bandwidth of the HBM; this kernel
// keeps 8 independent 16-byte loads per thread and ~1300 threads per SM in flight.
//
// The reference always runs with >= 2 ranks (its scripts assert `size > 1`, e.g. 6_allgather.py:186).
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch.h"

namespace mt {

constexpr int kCopyThreads = 256, kCopyUnroll = 8;

// src and dst share the same offset inside a 16-byte line (checked by the launcher): `head` single bytes bring
// both to a 16-byte boundary, then n16 vectors, then `tail` single bytes.
__global__ void __launch_bounds__(kCopyThreads) local_copy_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                                  uint32_t head, uint64_t n16, uint32_t tail) {
  const uint4* s = (const uint4*)(src + head);
  uint4* d = (uint4*)(dst + head);
  constexpr uint64_t kChunk = (uint64_t)kCopyThreads * kCopyUnroll;
  for (uint64_t base = (uint64_t)blockIdx.x * kChunk; base < n16; base += (uint64_t)gridDim.x * kChunk) {
    uint4 v[kCopyUnroll];
    if (base + kChunk <= n16) {
#pragma unroll
      for (int u = 0; u < kCopyUnroll; ++u) v[u] = __ldcs(s + base + u * kCopyThreads + threadIdx.x);
#pragma unroll
      for (int u = 0; u < kCopyUnroll; ++u) d[base + u * kCopyThreads + threadIdx.x] = v[u];
    } else {
#pragma unroll
      for (int u = 0; u < kCopyUnroll; ++u) {
        const uint64_t i = base + u * kCopyThreads + threadIdx.x;
        if (i < n16) v[u] = __ldcs(s + i);
      }
#pragma unroll
      for (int u = 0; u < kCopyUnroll; ++u) {
        const uint64_t i = base + u * kCopyThreads + threadIdx.x;
        if (i < n16) d[i] = v[u];
      }
    }
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x < head) dst[threadIdx.x] = src[threadIdx.x];
    if (threadIdx.x < tail) {
      const uint64_t o = (uint64_t)head + n16 * 16 + threadIdx.x;
      dst[o] = src[o];
    }
  }
}

// Returns cudaErrorInvalidValue when the two pointers sit at different offsets inside a 16-byte line (the caller
// then uses the general ring kernel).
cudaError_t launch_local_copy(void* dst, const void* src, uint64_t nbytes, int sms, cudaStream_t s) {
  if ((((uintptr_t)dst) ^ ((uintptr_t)src)) & 15) return cudaErrorInvalidValue;
  uint32_t head = (uint32_t)((16 - ((uintptr_t)src & 15)) & 15);
  if (head > nbytes) head = (uint32_t)nbytes;
  const uint64_t n16 = (nbytes - head) / 16;
  const uint32_t tail = (uint32_t)(nbytes - head - n16 * 16);
  const uint64_t chunks = (n16 + (uint64_t)kCopyThreads * kCopyUnroll - 1) / ((uint64_t)kCopyThreads * kCopyUnroll);
  uint64_t grid = chunks < 1 ? 1 : chunks;
  const uint64_t cap = (uint64_t)sms * 8;
  if (grid > cap) grid = cap;
  count_launch();
  local_copy_kernel<<<(unsigned)grid, kCopyThreads, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, head, n16, tail);
  return cudaGetLastError();
}

}  // namespace mt
