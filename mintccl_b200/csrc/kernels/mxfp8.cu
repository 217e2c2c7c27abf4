// Block-scaled fp8 (MXFP8: e4m3 payload, one ue8m0 scale per 32 elements) sum over ranks.
//
// Every rank holds a quantised tensor (payload bytes + scale bytes) in the symmetric heap.  The sum is
// formed in one hop: the owner of a 32-element block reads that block and its scale from every rank,
// dequantises, accumulates in fp32 in rank order (bit-identical on every rank), picks the new block scale
// from the block's largest magnitude and quantises once.  Intermediate hops of a ring would requantise
// n - 1 times; here precision is lost exactly once.  all-reduce writes the result to every rank
// (two-shot), reduce-scatter keeps the owner's shard.
//
// The reference only sums fp16 (primitive.py:230-247); fp8 is on its roadmap (README.md:58-60).
#include "../device/prims.cuh"
#include "../device/reduce_ops.cuh"
#include "../device/sched.h"
#include "launch.h"
#include "mxfp8.h"

namespace mt {

constexpr int kMxThreads = 256;

__device__ __forceinline__ void mx_accumulate(float* acc, u128 d0, u128 d1, uint8_t sc) {
  const float s = ue8m0_to_float(sc);
  const uint64_t w[4] = {d0.x, d0.y, d1.x, d1.y};
#pragma unroll
  for (int k = 0; k < 4; ++k)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[8 * k + b] += e4m3_to_float((uint8_t)(w[k] >> (8 * b))) * s;
}

__global__ void __launch_bounds__(kMxThreads, 2) mxfp8_kernel(const MtDevComm* comms, Mxfp8Args a) {
  __shared__ int s_fail;
  const int lr = blockIdx.y;
  const MtDevComm& c = comms[lr];
  const int n = c.nranks, me = c.rank;
  if (!rank_barrier(c, blockIdx.x, &s_fail)) return;
  // blocks this CTA works on, and inside them the ones this rank owns
  uint64_t lo, hi;
  if (a.op == MX_ALLREDUCE) {
    const MtRange r = mt_split(a.nblocks, gridDim.x, blockIdx.x, 1);
    const MtRange s = mt_split(r.hi - r.lo, n, me, 1);
    lo = r.lo + s.lo;
    hi = r.lo + s.hi;
  } else {
    const uint64_t per = a.nblocks / n;  // blocks per shard
    const MtRange r = mt_split(per, gridDim.x, blockIdx.x, 1);
    lo = (uint64_t)me * per + r.lo;
    hi = (uint64_t)me * per + r.hi;
  }
  for (uint64_t b = lo + threadIdx.x; b < hi; b += kMxThreads) {
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    for (int p = 0; p < n; ++p) {
      const uint8_t* dp = c.heap[p] + a.data_in_off + b * 32;
      const u128 d0 = load128_relaxed_sys(dp), d1 = load128_relaxed_sys(dp + 16);
      const uint8_t sc = *reinterpret_cast<const volatile uint8_t*>(c.heap[p] + a.scale_in_off + b);
      mx_accumulate(acc, d0, d1, sc);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(acc[i]));
    const uint8_t so = ue8m0_for_amax(amax);
    const float inv = 1.0f / ue8m0_to_float(so);
    uint64_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int q = 0; q < 8; ++q) w[k] |= (uint64_t)float_to_e4m3(acc[8 * k + q] * inv) << (8 * q);
    u128 o0, o1;
    o0.x = w[0]; o0.y = w[1]; o1.x = w[2]; o1.y = w[3];
    if (a.op == MX_ALLREDUCE) {
      for (int d = 0; d < n; ++d) {
        const int p = (me + d) % n;
        uint8_t* op_ = c.heap[p] + a.data_out_off + b * 32;
        store128_relaxed_sys(op_, o0);
        store128_relaxed_sys(op_ + 16, o1);
        *reinterpret_cast<volatile uint8_t*>(c.heap[p] + a.scale_out_off + b) = so;
      }
    } else {
      const uint64_t bl = b - (uint64_t)me * (a.nblocks / n);
      uint8_t* op_ = (uint8_t*)a.data_out[lr] + bl * 32;
      *reinterpret_cast<u128*>(op_) = o0;
      *reinterpret_cast<u128*>(op_ + 16) = o1;
      ((uint8_t*)a.scale_out[lr])[bl] = so;
    }
  }
  rank_barrier(c, blockIdx.x, &s_fail);
}

cudaError_t launch_mxfp8(const MtDevComm* comms, const Mxfp8Args& a, int nctas, int nlocal, cudaStream_t s) {
  Mxfp8Args args = a;
  void* p[] = {(void*)&comms, (void*)&args};
  return launch_any((const void*)mxfp8_kernel, dim3(nctas, nlocal), dim3(kMxThreads), p, s, nlocal > 1);
}

}  // namespace mt
