// Device intrinsics for peer-memory communication on sm_100a.
//
// Counterpart of the reference's primitive.py (thread_id, barrier_sync, syncwarp, syncthreads,
// threadfence, threadfence_system, any_sync, nanosleep, cvta_*, funnelshift_r, load128/store128,
// load64/store64 at primitive.py:20-227), extended with the qualifiers its docstring only plans
// (primitive.py:161-166: relaxed/acquire/release at system scope, L1::no_allocate streaming loads),
// NVLS multimem operations and bounded waits.  The reference's `trap` (primitive.py:116-120) has no
// counterpart on purpose: a failing wait records an error and returns, it never traps the GPU.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "layout.h"

namespace mt {

struct __align__(16) u128 {
  uint64_t x, y;
};

// ---- thread / warp / block helpers ----------------------------------------------------------------
__device__ __forceinline__ int thread_id() { return threadIdx.x; }
__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }
__device__ __forceinline__ void syncthreads() { __syncthreads(); }
__device__ __forceinline__ void syncwarp(unsigned mask = 0xffffffffu) { __syncwarp(mask); }
// Named barrier over `nthreads` threads (multiple of 32); id 0 is __syncthreads' barrier.
__device__ __forceinline__ void barrier_sync(int id, int nthreads) {
  asm volatile("barrier.sync.aligned %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ bool any_sync(bool pred, unsigned mask = 0xffffffffu) { return __any_sync(mask, pred); }
__device__ __forceinline__ void threadfence() { __threadfence(); }
__device__ __forceinline__ void threadfence_system() { __threadfence_system(); }
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void nanosleep(unsigned ns) { __nanosleep(ns); }
__device__ __forceinline__ uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t cvta_generic_to_shared(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void* cvta_shared_to_generic(uint32_t s) {
  uint64_t g;
  asm("{ .reg .u64 t; cvt.u64.u32 t, %1; cvta.shared.u64 %0, t; }" : "=l"(g) : "r"(s));
  return (void*)g;
}
__device__ __forceinline__ uint32_t funnelshift_r(uint32_t lo, uint32_t hi, uint32_t shift) {
  return __funnelshift_r(lo, hi, shift);
}

// ---- 128-bit and 64-bit global accesses ------------------------------------------------------------
// volatile: never cached in L1, never reordered with other volatile accesses of the thread.  Used for
// every access to memory that a peer writes behind our back (LL128 lines, FIFO slots).
__device__ __forceinline__ u128 load128(const void* p) {
  u128 v;
  asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store128(void* p, u128 v) {
  asm volatile("st.volatile.global.v2.u64 [%0], {%1,%2};" ::"l"(p), "l"(v.x), "l"(v.y) : "memory");
}
__device__ __forceinline__ uint64_t load64(const void* p) {
  uint64_t v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store64(void* p, uint64_t v) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Streaming read of data nobody modifies during the kernel (user inputs): read-only path, do not keep
// the line in L1.
__device__ __forceinline__ u128 load128_stream(const void* p) {
  u128 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p));
  return v;
}
// Relaxed system-scope accesses: coherent with peers, no ordering (bulk payload over NVLink).
__device__ __forceinline__ u128 load128_relaxed_sys(const void* p) {
  u128 v;
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store128_relaxed_sys(void* p, u128 v) {
  asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1,%2};" ::"l"(p), "l"(v.x), "l"(v.y) : "memory");
}
__device__ __forceinline__ uint64_t load64_acquire_sys(const void* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t load64_relaxed_sys(const void* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store64_release_sys(void* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void store64_relaxed_sys(void* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t load32_volatile(const void* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store32_relaxed_sys(void* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---- NVLS multimem (addresses are in the multicast alias of the heap) ------------------------------
struct __align__(16) f32x4 {
  float a, b, c, d;
};
__device__ __forceinline__ u128 multimem_ld_reduce_f32x4(const void* mc) {
  u128 v;
  uint32_t a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "l"(mc)
               : "memory");
  v.x = (uint64_t)a | ((uint64_t)b << 32);
  v.y = (uint64_t)c | ((uint64_t)d << 32);
  return v;
}
__device__ __forceinline__ u128 multimem_ld_reduce_bf16x8(const void* mc) {
  u128 v;
  uint32_t a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "l"(mc)
               : "memory");
  v.x = (uint64_t)a | ((uint64_t)b << 32);
  v.y = (uint64_t)c | ((uint64_t)d << 32);
  return v;
}
__device__ __forceinline__ u128 multimem_ld_reduce_f16x8(const void* mc) {
  u128 v;
  uint32_t a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "l"(mc)
               : "memory");
  v.x = (uint64_t)a | ((uint64_t)b << 32);
  v.y = (uint64_t)c | ((uint64_t)d << 32);
  return v;
}
__device__ __forceinline__ void multimem_st_128(void* mc, u128 v) {
  uint32_t a = (uint32_t)v.x, b = (uint32_t)(v.x >> 32), c = (uint32_t)v.y, d = (uint32_t)(v.y >> 32);
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

// ---- error reporting and bounded waits -------------------------------------------------------------
__device__ __forceinline__ MtStatus* status_of(const MtDevComm& c, int rank) {
  return (MtStatus*)(c.heap[rank] + c.L.status_off);
}

// Record the first error of this rank and raise the abort flag here and on every peer so that all
// other waits give up quickly instead of each running out its own time limit.
static __device__ __noinline__ void report_error(const MtDevComm& c, uint32_t code, uint32_t channel, uint32_t where,
                                          uint64_t expected, uint64_t seen, uint64_t step) {
  MtStatus* st = status_of(c, c.rank);
  if (atomicCAS(&st->code, 0u, code) == 0u) {
    st->rank = c.rank;
    st->channel = channel;
    st->where = where;
    st->expected = expected;
    st->seen = seen;
    st->step = step;
  }
  for (int p = 0; p < c.nranks; ++p) store32_relaxed_sys(&status_of(c, p)->abort, 1u);
  __threadfence_system();
}

__device__ __forceinline__ bool abort_raised(const MtDevComm& c) {
  return load32_volatile(&status_of(c, c.rank)->abort) != 0u;
}

// Spin until pred() holds.  Every 256 polls the abort flag and the wall-clock limit are checked; the
// wait backs off with nanosleep once it has clearly not been satisfied at once.  Returns false when it
// gave up (after recording the error); the caller must then unwind without touching peer memory again.
template <class Pred>
__device__ __forceinline__ bool bounded_wait(const MtDevComm& c, Pred pred, uint32_t code, uint32_t channel,
                                             uint32_t where, uint64_t expected, uint64_t step,
                                             const volatile uint64_t* seen_ptr) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!pred()) {
    ++spins;
    if ((spins & 0xffu) == 0u) {
      if (abort_raised(c)) {
        report_error(c, MT_ERR_REMOTE_ABORT, channel, where, expected, seen_ptr ? *seen_ptr : 0, step);
        return false;
      }
      uint64_t now = globaltimer();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > c.timeout_ns) {
        report_error(c, code, channel, where, expected, seen_ptr ? *seen_ptr : 0, step);
        return false;
      }
    }
    if (spins > 32u) __nanosleep(spins > 4096u ? 200u : 20u);
  }
  return true;
}

// ---- cross-rank barrier ----------------------------------------------------------------------------
// CTA `slot` of every rank meets the CTA with the same index on all other ranks.  Arrival counters
// only ever grow (the local epoch persists across kernels) so nothing is ever reset and a late or
// repeated store cannot be mistaken for a newer arrival.  The release store after the block barrier
// publishes every earlier store of the CTA; the acquire load orders every later access after the
// peers' arrivals.  `s_fail` is a shared-memory word used to make the outcome uniform in the CTA.
__device__ __forceinline__ bool rank_barrier(const MtDevComm& c, int slot, int* s_fail) {
  __syncthreads();
  MtBarSlot* mine = (MtBarSlot*)(c.heap[c.rank] + c.L.bar_off) + slot;
  const int t = threadIdx.x;
  if (t == 0) *s_fail = 0;
  __syncthreads();
  if (t < c.nranks) {
    uint64_t e = load64(&mine->epoch) + 1;
    fence_acq_rel_sys();
    MtBarSlot* theirs = (MtBarSlot*)(c.heap[t] + c.L.bar_off) + slot;
    store64_release_sys(&theirs->arrive[c.rank], e);
    const uint64_t* w = &mine->arrive[t];
    bool ok = bounded_wait(
        c, [&] { return load64_acquire_sys(w) >= e; }, MT_ERR_TIMEOUT_BARRIER, slot, MT_WHERE_BARRIER, e, 0,
        (const volatile uint64_t*)w);
    if (!ok) atomicExch(s_fail, 1);
  }
  __syncthreads();
  if (t == 0 && *s_fail == 0) store64(&mine->epoch, load64(&mine->epoch) + 1);
  __syncthreads();
  return *s_fail == 0;
}

// The same barrier, used as the entry barrier of a one-hop collective: with its arrival every rank also
// announces where its input and output buffers are, as seen from each peer.  Thread t < nranks talks to rank
// t, so `pub_in` / `pub_out` are per-thread values: what to announce to rank threadIdx.x (an address valid in
// that rank's address space, or MT_PUB_HEAP_TAG | offset inside my heap, or 0 for "none").
// On return `s_in[q]` / `s_out[q]` (shared memory, MT_MAX_RANKS entries) hold rank q's buffers as addresses
// that are valid here; entry `rank` holds `local_in` / `local_out`.  This is what lets the one-hop kernels
// run on ordinary device allocations registered through CUDA IPC, and on heap tensors whose offsets differ
// between ranks: nothing but this exchange depends on where a peer's buffer is.
__device__ __forceinline__ bool rank_barrier_xchg(const MtDevComm& c, int slot, int* s_fail, uint64_t pub_in,
                                                  uint64_t pub_out, const void* local_in, void* local_out,
                                                  const uint8_t** s_in, uint8_t** s_out) {
  __syncthreads();
  MtBarSlot* mine = (MtBarSlot*)(c.heap[c.rank] + c.L.bar_off) + slot;
  const int t = threadIdx.x;
  if (t == 0) *s_fail = 0;
  __syncthreads();
  if (t < c.nranks) {
    uint64_t e = load64(&mine->epoch) + 1;
    fence_acq_rel_sys();
    MtBarSlot* theirs = (MtBarSlot*)(c.heap[t] + c.L.bar_off) + slot;
    if (t != c.rank) {
      store64_relaxed_sys(&theirs->pin[c.rank], pub_in);
      store64_relaxed_sys(&theirs->pout[c.rank], pub_out);
    }
    store64_release_sys(&theirs->arrive[c.rank], e);
    const uint64_t* w = &mine->arrive[t];
    bool ok = bounded_wait(
        c, [&] { return load64_acquire_sys(w) >= e; }, MT_ERR_TIMEOUT_BARRIER, slot, MT_WHERE_BARRIER, e, 0,
        (const volatile uint64_t*)w);
    if (!ok) {
      atomicExch(s_fail, 1);
    } else if (t == c.rank) {
      s_in[t] = (const uint8_t*)local_in;
      s_out[t] = (uint8_t*)local_out;
    } else {
      const uint64_t vi = load64_relaxed_sys(&mine->pin[t]), vo = load64_relaxed_sys(&mine->pout[t]);
      s_in[t] = (vi & MT_PUB_HEAP_TAG) ? c.heap[t] + (vi & ~MT_PUB_HEAP_TAG) : (const uint8_t*)(uintptr_t)vi;
      s_out[t] = (vo & MT_PUB_HEAP_TAG) ? c.heap[t] + (vo & ~MT_PUB_HEAP_TAG) : (uint8_t*)(uintptr_t)vo;
    }
  }
  __syncthreads();
  if (t == 0 && *s_fail == 0) store64(&mine->epoch, load64(&mine->epoch) + 1);
  __syncthreads();
  return *s_fail == 0;
}

}  // namespace mt
