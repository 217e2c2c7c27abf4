// Direct point-to-point copy over a peer-mapped pointer, and the one-shot low-latency all-reduce.
//
// p2p: the reference's first script lets the receiver pull straight from the sender's buffer
// (1_sendrecv_direct.py:31-54) and relies on host-side MPI ordering alone; nothing tells the sender
// when its buffer may be reused.  Here both sides launch: the passive side announces "ready" and
// waits for "done", the copying side waits for "ready", moves the data with many 16-byte accesses in
// flight, and counts its CTAs into "done" with a release so the data is visible before the count.
//
// one-shot all-reduce: for messages of a few KiB the cost is latency, not bandwidth.  Every rank
// writes its contribution as LL128 lines (flag = call epoch) into a per-sender area of every peer and
// then sums what arrived; one kernel, no barrier, no host round trip, any input/output pointers.
#pragma once
#include "../device/proto_ll128.cuh"
#include "direct_engine.cuh"

namespace mt {

struct P2pArgs {
  const void* src[MT_MAX_RANKS];   // per local rank: the pointer the copying side reads
  void* dst[MT_MAX_RANKS];         // per local rank: the pointer the copying side writes
  uint64_t nbytes;
  int32_t role[MT_MAX_RANKS];      // per local rank: 0 none, 1 copier, 2 passive
  int32_t peer[MT_MAX_RANKS];      // per local rank: the other side
  uint64_t seq[MT_MAX_RANKS];      // ready sequence number of this transfer (per ordered pair)
  uint64_t done_target[MT_MAX_RANKS];  // cumulative CTA count the passive side waits for
  int32_t copier_reads_remote;     // pull (1): src is in the peer's memory; push (0): dst is
  int32_t mode;                    // how the payload moves: 0 system-scope relaxed 16-byte loads / stores,
                                   // 1 volatile loads and weak stores, 2 bulk copies staged in shared memory
};

// The same copy with the weakest qualifiers that are still correct for payload that is published by a later
// release: weak 16-byte stores, volatile (never L1-cached) loads of peer memory.
template <int NTHREADS, bool REMOTE_SRC>
__device__ __forceinline__ void copy_range_weak(const uint8_t* src, uint8_t* dst, uint64_t nbytes) {
  if ((((uintptr_t)src | (uintptr_t)dst) & 15) != 0) {
    copy_range<NTHREADS, REMOTE_SRC, !REMOTE_SRC>(src, dst, nbytes);
    return;
  }
  const uint64_t nvec = nbytes >> 4;
  constexpr int kU = 8;
  for (uint64_t base = 0; base < nvec; base += (uint64_t)NTHREADS * kU) {
    u128 v[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) v[u] = REMOTE_SRC ? load128(src + (i << 4)) : load128_stream(src + (i << 4));
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) *reinterpret_cast<u128*>(dst + (i << 4)) = v[u];
    }
  }
  for (uint64_t o = (nvec << 4) + threadIdx.x; o < nbytes; o += NTHREADS)
    *reinterpret_cast<volatile uint8_t*>(dst + o) = *reinterpret_cast<const volatile uint8_t*>(src + o);
}

__device__ __forceinline__ void red_release_sys_add_u64(uint64_t* p, uint64_t v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

template <int NTHREADS>
__global__ void __launch_bounds__(NTHREADS, 1) p2p_kernel(const MtDevComm* comms, P2pArgs a) {
  extern __shared__ uint8_t dyn_smem[];   // kBulkSmemBytes in mode 2
  __shared__ BulkCtl ctl;
  __shared__ int s_fail;
  const int lr = blockIdx.y;
  const MtDevComm& c = comms[lr];
  const int role = a.role[lr], peer = a.peer[lr];
  if (role == 0) return;
  MtSigSlot* mine = (MtSigSlot*)(c.heap[c.rank] + c.L.sig_off) + peer;       // words the peer writes
  MtSigSlot* theirs = (MtSigSlot*)(c.heap[peer] + c.L.sig_off) + c.rank;     // words I write
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (role == 2) {
    if (blockIdx.x != 0) return;
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      store64_release_sys(&theirs->ready, a.seq[lr]);
      const uint64_t want = a.done_target[lr];
      const uint64_t* w = &mine->done;
      bounded_wait(
          c, [&] { return load64_acquire_sys(w) >= want; }, MT_ERR_TIMEOUT_SIGNAL, 0, MT_WHERE_P2P_DONE, want, a.seq[lr],
          (const volatile uint64_t*)w);
    }
    return;
  }
  // copier
  if (threadIdx.x == 0) {
    const uint64_t want = a.seq[lr];
    const uint64_t* w = &mine->ready;
    if (!bounded_wait(
            c, [&] { return load64_acquire_sys(w) >= want; }, MT_ERR_TIMEOUT_SIGNAL, blockIdx.x, MT_WHERE_P2P_READY, want,
            a.seq[lr], (const volatile uint64_t*)w))
      s_fail = 1;
  }
  __syncthreads();
  if (s_fail) return;
  const MtRange r = mt_split(a.nbytes, gridDim.x, blockIdx.x, kSplitAlignDirect);
  const uint8_t* src = (const uint8_t*)a.src[lr];
  uint8_t* dst = (uint8_t*)a.dst[lr];
  if (r.hi > r.lo) {
    bool done = false;
    if (a.mode == 2 && ((((uintptr_t)src | (uintptr_t)dst) + r.lo) & 15) == 0) {
      if (threadIdx.x == 0) {
        ctl.jobs[0].src = src + r.lo;
        ctl.jobs[0].nbytes = (r.hi - r.lo) & ~15ull;
        ctl.jobs[0].ndst = 1;
        ctl.jobs[0].dst[0] = dst + r.lo;
        ctl.njobs = 1;
        uint8_t* ring = (uint8_t*)(((uintptr_t)dyn_smem + 1023) & ~(uintptr_t)1023);
        if (!bulk_run(&ctl, ring, c.timeout_ns)) {
          s_fail = 1;
          report_error(c, MT_ERR_TIMEOUT_FLAG, blockIdx.x, MT_WHERE_BULK, 0, 0, 0);
        }
      }
      const uint64_t tail = (r.hi - r.lo) & ~15ull;
      for (uint64_t o = r.lo + tail + threadIdx.x; o < r.hi; o += NTHREADS) *(volatile uint8_t*)(dst + o) = src[o];
      done = true;
    }
    if (!done) {
      if (a.mode == 1) {
        if (a.copier_reads_remote) copy_range_weak<NTHREADS, true>(src + r.lo, dst + r.lo, r.hi - r.lo);
        else copy_range_weak<NTHREADS, false>(src + r.lo, dst + r.lo, r.hi - r.lo);
      } else {
        if (a.copier_reads_remote) copy_range<NTHREADS, true, false>(src + r.lo, dst + r.lo, r.hi - r.lo);
        else copy_range<NTHREADS, false, true>(src + r.lo, dst + r.lo, r.hi - r.lo);
      }
    }
  }
  __syncthreads();
  if (s_fail) return;
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    red_release_sys_add_u64(&theirs->done, 1);
  }
}

// ---- one-shot LL128 all-reduce ---------------------------------------------------------------------
struct LLArgs {
  const void* in[MT_MAX_RANKS];
  void* out[MT_MAX_RANKS];
  uint64_t nbytes;   // <= payload capacity of the one-shot area
};

// grid.x CTAs split the warp chunks of the message; epoch (one per CTA) grows by one per call.
template <class T, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS, 1) ll_allreduce_kernel(const MtDevComm* comms, LLArgs a) {
  __shared__ int s_fail;
  const int lr = blockIdx.y;
  const MtDevComm& c = comms[lr];
  const int n = c.nranks, me = c.rank;
  if (threadIdx.x == 0) s_fail = 0;
  uint64_t* epoch_ptr = (uint64_t*)(c.heap[me] + c.L.ll_epoch_off) + blockIdx.x;
  const uint64_t epoch = load64(epoch_ptr) + 1;
  __syncthreads();
  const uint64_t parity = epoch & 1;
  const uint8_t* in = (const uint8_t*)a.in[lr];
  uint8_t* out = (uint8_t*)a.out[lr];
  const bool in_al = ((uintptr_t)in & 15) == 0, out_al = ((uintptr_t)out & 15) == 0;
  const uint32_t nchunks = (uint32_t)mt_div_up(a.nbytes, MT_LL128_WARP_PAYLOAD);
  const uint32_t warps_total = gridDim.x * (NTHREADS / 32);
  bool ok = true;
  for (uint32_t wc = blockIdx.x * (NTHREADS / 32) + (threadIdx.x >> 5); ok && wc < nchunks; wc += warps_total) {
    const uint64_t po = (uint64_t)wc * MT_LL128_WARP_PAYLOAD, wo = (uint64_t)wc * MT_LL128_WARP_WIRE;
    const uint64_t left = a.nbytes - po;
    const int nb = left < MT_LL128_WARP_PAYLOAD ? (int)left : MT_LL128_WARP_PAYLOAD;
    const LL128Lane L(nb);
    uint64_t mineb[8];
    ll128_load_raw(L, in + po, nb, in_al, mineb);
    // push my lines to every peer's area for me
    for (int d = 1; d < n; ++d) {
      const int p = (me + d) % n;
      uint8_t* wire = c.heap[p] + c.L.ll_off + (parity * n + me) * c.L.ll_bytes + wo;
      ll128_store_wire(L, wire, mineb, epoch);
    }
    // sum in rank order so that every rank computes bit-identical results
    float acc[8][T::kPer64];
#pragma unroll
    for (int w = 0; w < 8; ++w)
#pragma unroll
      for (int e = 0; e < T::kPer64; ++e) acc[w][e] = 0.f;
    auto add = [&](const uint64_t* v) {
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        if (L.flag_lane && (w & 1)) continue;  // flag words carry no payload
        float f[T::kPer64];
        T::unpack(v[w], f);
#pragma unroll
        for (int e = 0; e < T::kPer64; ++e) acc[w][e] += f[e];
      }
    };
    // The peers' lines arrive at about the same time, so they are polled four ranks at a time: the loads of a
    // whole group are in flight together (one round trip to the L2 per group instead of one per rank).
    const uint8_t* area = c.heap[me] + c.L.ll_off + (parity * n) * c.L.ll_bytes + wo;
    for (int g0 = 0; g0 < n && ok; g0 += 4) {
      uint64_t v[4][8];
      unsigned pending = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (g0 + j < n && g0 + j != me) pending |= 1u << j;
      uint32_t spins = 0;
      uint64_t t0 = 0;
      while (pending) {
        bool bad[4] = {false, false, false, false};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (pending & (1u << j)) {
            const uint8_t* wire = area + (uint64_t)(g0 + j) * c.L.ll_bytes;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (L.need[k]) {
                const u128 t = load128(wire + L.wire_off(k));
                v[j][2 * k] = t.x;
                v[j][2 * k + 1] = t.y;
                if (L.flag_lane && t.y != epoch) bad[j] = true;
              }
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if ((pending & (1u << j)) && !__any_sync(0xffffffffu, bad[j])) pending &= ~(1u << j);
        if (!pending) break;
        if ((++spins & 0xffu) == 0u) {
          int giveup = 0;
          if ((threadIdx.x & 31) == 0) {
            if (abort_raised(c) || *(volatile int*)&s_fail) {
              giveup = MT_ERR_REMOTE_ABORT;
            } else {
              const uint64_t now = globaltimer();
              if (t0 == 0) t0 = now;
              else if (now - t0 > c.timeout_ns) giveup = MT_ERR_TIMEOUT_FLAG;
            }
          }
          giveup = __shfl_sync(0xffffffffu, giveup, 0);
          if (giveup) {
            if ((threadIdx.x & 31) == 0) {
              report_error(c, giveup, blockIdx.x, MT_WHERE_LL_ONESHOT, epoch, 0, epoch);
              atomicExch(&s_fail, 1);
            }
            ok = false;
            break;
          }
        }
        if (spins > 32u) __nanosleep(20);
      }
      if (!ok) break;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (g0 + j >= n) break;
        if (g0 + j == me) add(mineb);
        else add(v[j]);
      }
    }
    if (ok) {
      uint64_t r[8];
#pragma unroll
      for (int w = 0; w < 8; ++w) r[w] = T::pack(acc[w]);
      ll128_store_raw(L, out + po, nb, out_al, r);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && s_fail == 0) store64(epoch_ptr, epoch);
}

}  // namespace mt
