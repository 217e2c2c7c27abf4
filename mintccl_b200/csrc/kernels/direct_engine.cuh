// One-hop collectives for fully connected (NVSwitch) nodes, and their NVLS multimem variants.
//
// The reference only has ring algorithms (README.md:53-55) because it targets machines without a
// switch; on B200 every peer is one hop away at full bandwidth, so for most sizes the fastest
// schedule is "everybody talks to everybody at once": all-gather pushes a shard to every peer,
// reduce-scatter pulls one shard from every peer and sums in fp32 registers, all-reduce does both
// ("two-shot"), all-to-all pushes block p to peer p.  With NVLS the switch does the summing
// (multimem.ld_reduce) and the replication (multimem.st).
//
// Buffers that peers touch must live in the symmetric heap (same offset on every rank).  CTA i of
// every rank works on the same slice of the message, so the only cross-rank dependencies are between
// CTAs with equal index; each CTA brackets its work with a bounded cross-rank barrier on its slot.
#pragma once
#include "../device/proto_ll128.cuh"

namespace mt {

enum DirectOp : int {
  DOP_ALLGATHER = 0,      // in: local shard; out: symmetric [n][B]
  DOP_REDUCESCATTER = 1,  // in: symmetric [n][B]; out: local shard
  DOP_ALLREDUCE = 2,      // in: symmetric N; out: symmetric N (two-shot) or local (one-shot)
  DOP_ALLTOALL = 3,       // in: local [n][B]; out: symmetric [n][B]
  DOP_BROADCAST = 4,      // in: root local; out: symmetric
  DOP_REDUCE = 5,         // in: symmetric; out: root local
};

struct DirectArgs {
  const void* in[MT_MAX_RANKS];  // local view of the input, per local rank
  void* out[MT_MAX_RANKS];       // local view of the output, per local rank
  uint64_t in_off;               // heap offset of the input when peers read it
  uint64_t out_off;              // heap offset of the output when peers write it
  uint64_t nbytes;               // AG/RS/A2A: bytes per shard; others: message bytes
  int32_t op;
  int32_t root;
  int32_t variant;               // all-reduce: 0 two-shot, 1 one-shot; all-gather/all-to-all: 0 push, 1 pull;
                                 // broadcast: 0 root pushes, 1 peers pull, 2 pull + replicate (every rank reads 1/n from the root and stores it to all);
                                 // reduce: 0 root sums, 2 reduce-scatter + gather into the root
  int32_t nvls;                  // use multimem instructions
};

static constexpr int kDirectUnroll = 4;

// Alignment of the boundaries between the slices of different CTAs.
static constexpr uint64_t kSplitAlignDirect = 128;

// out[i] = sum over ranks of peer_in[rank][i] for message bytes [byte_lo, byte_hi); the result is
// stored to `local_out` and, if PUSH, to the same offset of every peer's output.  Offset o of the
// message lands at local_out + (o - local_base).  FIXED_ORDER sums ranks 0..n-1 in that order on every
// rank (bitwise identical results everywhere, needed when several ranks reduce the same element);
// otherwise each rank starts at itself so that the n readers spread over the n memories.
template <class T, int NTHREADS, bool PUSH, bool FIXED_ORDER, int NR>
__device__ __forceinline__ void pull_reduce_range_n(const MtDevComm& c, uint64_t in_off, uint64_t out_off,
                                                    uint8_t* local_out, uint64_t byte_lo, uint64_t byte_hi,
                                                    uint64_t local_base) {
  // NR > 0: the rank count is a compile-time constant, so the loop over peers unrolls and all
  // NR x kU remote loads of a thread are in flight together
  const int n = NR > 0 ? NR : c.nranks;
  // vectors per thread and pass: bounded so that NR x kU 16-byte registers fit without spilling
  constexpr int kU = NR >= 8 ? 2 : kDirectUnroll;
  // 16-byte vectors need every address involved to be 16-byte aligned; heaps are, so only the offsets
  // count (a shard offset rank * B is unaligned when B is not a multiple of 16).
  const bool vec_ok = (((in_off + byte_lo) | (PUSH ? out_off + byte_lo : 0) |
                        (uint64_t)(uintptr_t)(local_out + (byte_lo - local_base))) & 15) == 0;
  const uint64_t nvec = vec_ok ? (byte_hi - byte_lo) >> 4 : 0;
  for (uint64_t base = 0; base < nvec; base += (uint64_t)NTHREADS * kU) {
    Acc128<T> acc[kU];
    if (NR > 0) {
      u128 v[NR > 0 ? NR : 1][kU];
#pragma unroll
      for (int d = 0; d < NR; ++d) {
        const int p = FIXED_ORDER ? d : (c.rank + d) % NR;
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
          if (i < nvec) v[d][u] = load128_relaxed_sys(c.heap[p] + in_off + byte_lo + (i << 4));
        }
      }
#pragma unroll
      for (int d = 0; d < NR; ++d) {
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          if (d == 0) acc[u].set(v[d][u]);
          else acc[u].add(v[d][u]);
        }
      }
    } else {
      u128 v[kU];
      for (int d = 0; d < n; ++d) {
        const int p = FIXED_ORDER ? d : (c.rank + d) % n;
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
          if (i < nvec) v[u] = load128_relaxed_sys(c.heap[p] + in_off + byte_lo + (i << 4));
        }
        if (d == 0) {
#pragma unroll
          for (int u = 0; u < kU; ++u) acc[u].set(v[u]);
        } else {
#pragma unroll
          for (int u = 0; u < kU; ++u) acc[u].add(v[u]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) {
        const u128 r = acc[u].get();
        const uint64_t o = byte_lo + (i << 4);
        *reinterpret_cast<u128*>(local_out + (o - local_base)) = r;
        if (PUSH) {
          for (int d = 1; d < n; ++d) {
            const int p = (c.rank + d) % n;
            store128_relaxed_sys(c.heap[p] + out_off + o, r);
          }
        }
      }
    }
  }
  // what the vectors did not cover (a tail of < 16 bytes, or everything when unaligned), element-wise
  using E = typename T::elem;
  const uint64_t done = byte_lo + (nvec << 4);
  const uint64_t nel = (byte_hi - done) / sizeof(E);
  for (uint64_t e_i = threadIdx.x; e_i < nel; e_i += NTHREADS) {
    const uint64_t o = done + e_i * sizeof(E);
    float acc = 0.f;
    for (int d = 0; d < n; ++d) {
      const int p = FIXED_ORDER ? d : (c.rank + d) % n;
      const E x = *reinterpret_cast<const volatile E*>(c.heap[p] + in_off + o);
      acc += elem_to_float<T>(x);
    }
    const E e = float_to_elem<T>(acc);
    *reinterpret_cast<E*>(local_out + (o - local_base)) = e;
    if (PUSH)
      for (int d = 1; d < n; ++d) *reinterpret_cast<volatile E*>(c.heap[(c.rank + d) % n] + out_off + o) = e;
  }
}

template <class T, int NTHREADS, bool PUSH, bool FIXED_ORDER>
__device__ __forceinline__ void pull_reduce_range(const MtDevComm& c, uint64_t in_off, uint64_t out_off,
                                                  uint8_t* local_out, uint64_t byte_lo, uint64_t byte_hi,
                                                  uint64_t local_base) {
  switch (c.nranks) {
    case 2: pull_reduce_range_n<T, NTHREADS, PUSH, FIXED_ORDER, 2>(c, in_off, out_off, local_out, byte_lo, byte_hi, local_base); break;
    case 4: pull_reduce_range_n<T, NTHREADS, PUSH, FIXED_ORDER, 4>(c, in_off, out_off, local_out, byte_lo, byte_hi, local_base); break;
    case 8: pull_reduce_range_n<T, NTHREADS, PUSH, FIXED_ORDER, 8>(c, in_off, out_off, local_out, byte_lo, byte_hi, local_base); break;
    default: pull_reduce_range_n<T, NTHREADS, PUSH, FIXED_ORDER, 0>(c, in_off, out_off, local_out, byte_lo, byte_hi, local_base); break;
  }
}

// Copy [lo, hi) bytes from src to dst with 16-byte vectors (+ byte tail).  REMOTE_SRC / REMOTE_DST
// select system-scope accesses for the side that lives in a peer's memory.
template <int NTHREADS, bool REMOTE_SRC, bool REMOTE_DST>
__device__ __forceinline__ void copy_range(const uint8_t* src, uint8_t* dst, uint64_t nbytes) {
  if ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
    const uint64_t nvec = nbytes >> 4;
    for (uint64_t base = 0; base < nvec; base += (uint64_t)NTHREADS * kDirectUnroll) {
      u128 v[kDirectUnroll];
#pragma unroll
      for (int u = 0; u < kDirectUnroll; ++u) {
        const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
        if (i < nvec) v[u] = REMOTE_SRC ? load128_relaxed_sys(src + (i << 4)) : load128_stream(src + (i << 4));
      }
#pragma unroll
      for (int u = 0; u < kDirectUnroll; ++u) {
        const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
        if (i < nvec) {
          if (REMOTE_DST) store128_relaxed_sys(dst + (i << 4), v[u]);
          else *reinterpret_cast<u128*>(dst + (i << 4)) = v[u];
        }
      }
    }
    for (uint64_t o = (nvec << 4) + threadIdx.x; o < nbytes; o += NTHREADS)
      *reinterpret_cast<volatile uint8_t*>(dst + o) = *reinterpret_cast<const volatile uint8_t*>(src + o);
  } else {
    for (uint64_t o = threadIdx.x; o < nbytes; o += NTHREADS)
      *reinterpret_cast<volatile uint8_t*>(dst + o) = *reinterpret_cast<const volatile uint8_t*>(src + o);
  }
}

template <class T>
__device__ __forceinline__ u128 mc_ld_reduce(const void* p);
template <>
__device__ __forceinline__ u128 mc_ld_reduce<F32>(const void* p) { return multimem_ld_reduce_f32x4(p); }
template <>
__device__ __forceinline__ u128 mc_ld_reduce<F16>(const void* p) { return multimem_ld_reduce_f16x8(p); }
template <>
__device__ __forceinline__ u128 mc_ld_reduce<BF16>(const void* p) { return multimem_ld_reduce_bf16x8(p); }
template <>
__device__ __forceinline__ u128 mc_ld_reduce<U8>(const void* p) { return load128(p); }

// NVLS loops with several multimem operations in flight per thread (a multimem round trip through the
// switch is several microseconds, so the depth matters more than for plain peer loads).
static constexpr int kNvlsUnroll = 4;
// dst[i] = sum over all ranks of mc_src[i]; dst is local memory, or the multicast alias when TO_MC.
template <class T, int NTHREADS, bool TO_MC>
__device__ __forceinline__ void nvls_reduce_range(const uint8_t* mc_src, uint8_t* dst, uint64_t nvec) {
  for (uint64_t base = 0; base < nvec; base += (uint64_t)NTHREADS * kNvlsUnroll) {
    u128 v[kNvlsUnroll];
#pragma unroll
    for (int u = 0; u < kNvlsUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) v[u] = mc_ld_reduce<T>(mc_src + (i << 4));
    }
#pragma unroll
    for (int u = 0; u < kNvlsUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) {
        if (TO_MC) multimem_st_128(dst + (i << 4), v[u]);
        else *reinterpret_cast<u128*>(dst + (i << 4)) = v[u];
      }
    }
  }
}
// mc_dst[i] (every rank's copy) = src[i]
// COHERENT: src was written by a peer during this kernel, so it must not go through the read-only path.
template <int NTHREADS, bool COHERENT = false>
__device__ __forceinline__ void nvls_bcast_range(const uint8_t* src, uint8_t* mc_dst, uint64_t nvec) {
  for (uint64_t base = 0; base < nvec; base += (uint64_t)NTHREADS * kNvlsUnroll) {
    u128 v[kNvlsUnroll];
#pragma unroll
    for (int u = 0; u < kNvlsUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) v[u] = COHERENT ? load128_relaxed_sys(src + (i << 4)) : load128_stream(src + (i << 4));
    }
#pragma unroll
    for (int u = 0; u < kNvlsUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) multimem_st_128(mc_dst + (i << 4), v[u]);
    }
  }
}

// dst_off of every peer (and local_dst unless skip_local) = src, reading each vector once.
template <int NTHREADS>
__device__ __forceinline__ void bcast_fanout(const MtDevComm& c, const uint8_t* src, uint64_t dst_off, uint8_t* local_dst,
                                             uint64_t nbytes, bool skip_local) {
  const int n = c.nranks;
  const uint64_t nvec = nbytes >> 4;
  for (uint64_t base = 0; base < nvec; base += (uint64_t)NTHREADS * kDirectUnroll) {
    u128 v[kDirectUnroll];
#pragma unroll
    for (int u = 0; u < kDirectUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) v[u] = load128_relaxed_sys(src + (i << 4));
    }
#pragma unroll
    for (int u = 0; u < kDirectUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) {
        for (int d = 1; d < n; ++d) store128_relaxed_sys(c.heap[(c.rank + d) % n] + dst_off + (i << 4), v[u]);
        if (!skip_local) *reinterpret_cast<u128*>(local_dst + (i << 4)) = v[u];
      }
    }
  }
}

template <class T, int NTHREADS>
__device__ void direct_body(const MtDevComm& c, const DirectArgs& a, int lr, int cta, int ncta, int* s_fail) {
  const int n = c.nranks, me = c.rank;
  const uint8_t* in = (const uint8_t*)a.in[lr];
  uint8_t* out = (uint8_t*)a.out[lr];
  const uint64_t B = a.nbytes;

  if (!rank_barrier(c, cta, s_fail)) return;

  switch (a.op) {
    case DOP_ALLGATHER: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (r.hi > r.lo) {
        if (a.nvls) {
          // one multimem store lands in every rank's output (mine included)
          uint8_t* mdst = c.mc + a.out_off + (uint64_t)me * B;
          const uint64_t nvec = (r.hi - r.lo) >> 4;
          nvls_bcast_range<NTHREADS>(in + r.lo, mdst + r.lo, nvec);
          // a tail cannot be sent with 16-byte multimem stores
          for (uint64_t o = r.lo + (nvec << 4) + threadIdx.x; o < r.hi; o += NTHREADS)
            for (int p = 0; p < n; ++p) *(volatile uint8_t*)(c.heap[p] + a.out_off + (uint64_t)me * B + o) = in[o];
        } else if (a.variant == 0) {
          for (int d = 0; d < n; ++d) {
            const int p = (me + d) % n;
            uint8_t* dst = (p == me ? out : c.heap[p] + a.out_off) + (uint64_t)me * B;
            if (p == me && in == dst) continue;
            copy_range<NTHREADS, false, true>(in + r.lo, dst + r.lo, r.hi - r.lo);
          }
        } else {
          for (int d = 0; d < n; ++d) {
            const int p = (me + d) % n;
            if (p == me) {
              if (in != out + (uint64_t)me * B) copy_range<NTHREADS, false, false>(in + r.lo, out + (uint64_t)me * B + r.lo, r.hi - r.lo);
            } else {
              // in_off == ~0: every rank's contribution is row `rank` of its own (symmetric) output buffer
              const uint64_t src_off = a.in_off == ~0ull ? a.out_off + (uint64_t)p * B : a.in_off;
              copy_range<NTHREADS, true, false>(c.heap[p] + src_off + r.lo, out + (uint64_t)p * B + r.lo, r.hi - r.lo);
            }
          }
        }
      }
      break;
    }
    case DOP_ALLTOALL: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (r.hi > r.lo) {
        for (int d = 0; d < n; ++d) {
          const int p = (me + d) % n;
          if (a.variant == 0) {  // push block p of my input into slot `me` of p's output
            uint8_t* dst = (p == me ? out : c.heap[p] + a.out_off) + (uint64_t)me * B;
            copy_range<NTHREADS, false, true>(in + (uint64_t)p * B + r.lo, dst + r.lo, r.hi - r.lo);
          } else {  // pull block `me` of p's input into slot p of my output
            const uint8_t* src = (p == me ? in : c.heap[p] + a.in_off) + (uint64_t)me * B;
            copy_range<NTHREADS, true, false>(src + r.lo, out + (uint64_t)p * B + r.lo, r.hi - r.lo);
          }
        }
      }
      break;
    }
    case DOP_REDUCESCATTER: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (r.hi > r.lo) {
        const uint64_t so = (uint64_t)me * B;
        if (a.nvls) {
          const uint8_t* msrc = c.mc + a.in_off + so;
          const uint64_t nvec = (r.hi - r.lo) >> 4;
          nvls_reduce_range<T, NTHREADS, false>(msrc + r.lo, out + r.lo, nvec);
          if (r.lo + (nvec << 4) < r.hi)
            pull_reduce_range<T, NTHREADS, false, false>(c, a.in_off, 0, out, so + r.lo + (nvec << 4), so + r.hi, so);
        } else {
          pull_reduce_range<T, NTHREADS, false, false>(c, a.in_off, 0, out, so + r.lo, so + r.hi, so);
        }
      }
      break;
    }
    case DOP_ALLREDUCE: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (r.hi > r.lo) {
        if (a.variant == 1) {  // one-shot: everybody sums everything, writes locally only
          pull_reduce_range<T, NTHREADS, false, true>(c, a.in_off, 0, out, r.lo, r.hi, 0);
        } else {
          // two-shot: inside this CTA's slice, rank `me` owns sub-slice `me`
          const MtRange s = mt_split(r.hi - r.lo, n, me, 16);
          const uint64_t lo = r.lo + s.lo, hi = r.lo + s.hi;
          if (hi > lo) {
            if (a.nvls) {
              const uint64_t nvec = (hi - lo) >> 4;
              nvls_reduce_range<T, NTHREADS, true>(c.mc + a.in_off + lo, c.mc + a.out_off + lo, nvec);
              if (lo + (nvec << 4) < hi)
                pull_reduce_range<T, NTHREADS, true, false>(c, a.in_off, a.out_off, out, lo + (nvec << 4), hi, 0);
            } else {
              pull_reduce_range<T, NTHREADS, true, false>(c, a.in_off, a.out_off, out, lo, hi, 0);
            }
          }
        }
      }
      break;
    }
    case DOP_BROADCAST: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (a.variant == 2) {
        // pull + replicate: rank j fetches sub-slice j straight from the root's buffer and replicates it
        // to everybody (one multimem.st per vector, or plain stores to every peer).  The root's link only
        // carries each byte once, the replication is spread over all ranks (a single source of multicast
        // stores tops out near 400 GB/s), and there is no phase in which only the root's link is busy.
        const uint64_t len = r.hi - r.lo;
        const MtRange sm = mt_split(len, n, me, 16);
        if (sm.hi > sm.lo) {
          const uint8_t* src = (me == a.root ? in : c.heap[a.root] + a.in_off) + r.lo + sm.lo;
          const uint64_t nb = sm.hi - sm.lo;
          if (a.nvls) {
            if (me == a.root) nvls_bcast_range<NTHREADS, false>(src, c.mc + a.out_off + r.lo + sm.lo, nb >> 4);
            else nvls_bcast_range<NTHREADS, true>(src, c.mc + a.out_off + r.lo + sm.lo, nb >> 4);
          } else {
            bcast_fanout<NTHREADS>(c, src, a.out_off + r.lo + sm.lo, out + r.lo + sm.lo, nb, me == a.root && in == out);
          }
        }
        break;
      }
      if (r.hi > r.lo) {
        if (a.nvls) {
          if (me == a.root) {
            const uint64_t nvec = (r.hi - r.lo) >> 4;
            nvls_bcast_range<NTHREADS>(in + r.lo, c.mc + a.out_off + r.lo, nvec);
            for (uint64_t o = r.lo + (nvec << 4) + threadIdx.x; o < r.hi; o += NTHREADS)
              for (int p = 0; p < n; ++p) *(volatile uint8_t*)(c.heap[p] + a.out_off + o) = in[o];
          }
        } else if (a.variant == 0) {
          if (me == a.root) {
            for (int d = 0; d < n; ++d) {
              const int p = (me + d) % n;
              uint8_t* dst = (p == me ? out : c.heap[p] + a.out_off);
              if (p == me && in == out) continue;
              copy_range<NTHREADS, false, true>(in + r.lo, dst + r.lo, r.hi - r.lo);
            }
          }
        } else {
          if (me != a.root) copy_range<NTHREADS, true, false>(c.heap[a.root] + a.in_off + r.lo, out + r.lo, r.hi - r.lo);
          else if (in != out) copy_range<NTHREADS, false, false>(in + r.lo, out + r.lo, r.hi - r.lo);
        }
      }
      break;
    }
    case DOP_REDUCE: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (a.variant == 2) {
        // reduce-scatter + gather: rank j sums sub-slice j (in the switch, or by pulling from every peer)
        // and stores the result straight into the root's output, so the summing is spread over all ranks
        // and the root only receives.
        const MtRange sm = mt_split(r.hi - r.lo, n, me, 16);
        if (sm.hi > sm.lo) {
          const uint64_t lo = r.lo + sm.lo, hi = r.lo + sm.hi;
          uint8_t* dst = me == a.root ? out : c.heap[a.root] + a.out_off;
          if (a.nvls) {
            nvls_reduce_range<T, NTHREADS, false>(c.mc + a.in_off + lo, dst + lo, (hi - lo) >> 4);
          } else {
            pull_reduce_range<T, NTHREADS, false, false>(c, a.in_off, 0, dst, lo, hi, 0);
          }
        }
        break;
      }
      if (a.variant == 3) {
        // the root only receives: the other n - 1 ranks each sum one sub-slice (pulling it from everybody,
        // the root included) and store the result into the root's output.  Every link then carries about
        // one message size, where "root sums everything" puts (n - 1) messages on the root's link.
        if (me != a.root) {
          const int idx = mt_mod(me - a.root - 1, n);
          const MtRange sm = mt_split(r.hi - r.lo, n - 1, idx, 16);
          if (sm.hi > sm.lo)
            pull_reduce_range<T, NTHREADS, false, false>(c, a.in_off, 0, c.heap[a.root] + a.out_off, r.lo + sm.lo,
                                                         r.lo + sm.hi, 0);
        }
        break;
      }
      if (r.hi > r.lo && me == a.root) {
        if (a.nvls) {
          const uint64_t nvec = (r.hi - r.lo) >> 4;
          nvls_reduce_range<T, NTHREADS, false>(c.mc + a.in_off + r.lo, out + r.lo, nvec);
          if (r.lo + (nvec << 4) < r.hi)
            pull_reduce_range<T, NTHREADS, false, false>(c, a.in_off, 0, out, r.lo + (nvec << 4), r.hi, 0);
        } else {
          pull_reduce_range<T, NTHREADS, false, false>(c, a.in_off, 0, out, r.lo, r.hi, 0);
        }
      }
      break;
    }
    default: break;
  }

  rank_barrier(c, cta, s_fail);
}

template <class T, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS, 1) direct_kernel(const MtDevComm* comms, DirectArgs a) {
  __shared__ int s_fail;
  const int lr = blockIdx.y;
  direct_body<T, NTHREADS>(comms[lr], a, lr, blockIdx.x, gridDim.x, &s_fail);
}

}  // namespace mt
