// One-hop collectives for fully connected (NVSwitch) nodes, and their NVLS multimem variants.
//
// The reference only has ring algorithms (README.md:53-55) because it targets machines without a
// switch; on B200 every peer is one hop away at full bandwidth, so for most sizes the fastest
// schedule is "everybody talks to everybody at once": all-gather pushes a shard to every peer,
// reduce-scatter pulls one shard from every peer and sums in fp32 registers, all-reduce does both
// ("two-shot"), all-to-all pushes block p to peer p.  With NVLS the switch does the summing
// (multimem.ld_reduce) and the replication (multimem.st).
//
// Buffers that peers touch must be mapped by the peers: tensors of the symmetric heap (any offset), or
// ordinary device allocations registered through CUDA IPC.  Where they are is announced rank to rank with
// the arrival at the entry barrier (rank_barrier_xchg), so the kernels only ever see "rank q's input /
// output as an address valid here".  The NVLS variants go through the multicast alias of the heap and
// therefore need heap tensors at the same offset on every rank.  CTA i of every rank works on the same
// slice of the message, so the only cross-rank dependencies are between CTAs with equal index; each CTA
// brackets its work with a bounded cross-rank barrier on its slot.
//
// The reducing operations are templated on the element type of the input and of the output: 16-bit input
// with fp32 output and fp32 input with 16-bit output sum in fp32 registers and round once, into the output
// type (the reference sums fp16 into fp16 only, primitive.py:230-247; other types are on its roadmap,
// README.md:58-60).  Byte counts and offsets are in input bytes throughout.
#pragma once
#include <type_traits>
#include "../device/proto_ll128.cuh"
#include "../device/tc_prims.cuh"

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
  uint64_t pub_in[MT_MAX_RANKS];   // what this rank announces to peer p as its input (see rank_barrier_xchg)
  uint64_t pub_out[MT_MAX_RANKS];  // ... and as its output
  uint64_t mc_in_off;            // NVLS: heap offset of the input (the same on every rank)
  uint64_t mc_out_off;           // NVLS: heap offset of the output
  uint64_t nbytes;               // AG/RS/A2A: bytes per shard; others: message bytes (input bytes)
  int32_t op;
  int32_t root;
  int32_t variant;               // all-reduce: 0 two-shot, 1 one-shot; all-gather/all-to-all: 0 push, 1 pull, 4 bulk push, 5 bulk pull (all-gather);
                                 // broadcast: 4 bulk pull + replicate (the copy engine variants need dynamic shared memory);
                                 // broadcast: 0 root pushes, 1 peers pull, 2 pull + replicate (every rank reads 1/n from the root and stores it to all);
                                 // reduce: 0 root sums, 2 NVLS reduce-scatter + gather into the root, 3 the others sum and store into the root
  int32_t nvls;                  // use multimem instructions
  int32_t pub_local;             // one address space (emulated world): announce in[] / out[] themselves
};

// Element types of a reducing kernel: input TI, output TO.
template <class TI, class TO>
struct CastInfo {
  static constexpr bool kSame = std::is_same<TI, TO>::value;
  static constexpr int kSI = (int)sizeof(typename TI::elem), kSO = (int)sizeof(typename TO::elem);
  static_assert(kSame || (kSI == 2 && kSO == 4) || (kSI == 4 && kSO == 2), "16-bit <-> fp32 only");
  // output byte offset of the element that starts at input byte offset o
  static __device__ __forceinline__ uint64_t out_off(uint64_t o) { return kSame ? o : (kSI == 2 ? o * 2 : o / 2); }
  // alignment the output address of a 16-byte input vector needs
  static constexpr uint64_t kOutAlignMask = (!kSame && kSI == 4) ? 7 : 15;
};

// Store the fp32 sums of one 16-byte input vector at input offset o of the message whose output starts at
// `out_base`, rounded once into TO.
template <class TI, class TO, bool REMOTE>
__device__ __forceinline__ void store_acc(uint8_t* out_base, uint64_t o, const Acc128<TI>& acc) {
  using CI = CastInfo<TI, TO>;
  if constexpr (CI::kSame) {
    const u128 r = acc.get();
    if (REMOTE) store128_relaxed_sys(out_base + o, r);
    else *reinterpret_cast<u128*>(out_base + o) = r;
  } else if constexpr (CI::kSI == 2) {  // 8 sums -> 32 bytes of fp32
    u128 lo, hi;
    lo.x = F32::pack(acc.f);
    lo.y = F32::pack(acc.f + 2);
    hi.x = F32::pack(acc.f + 4);
    hi.y = F32::pack(acc.f + 6);
    uint8_t* d = out_base + o * 2;
    if (REMOTE) {
      store128_relaxed_sys(d, lo);
      store128_relaxed_sys(d + 16, hi);
    } else {
      *reinterpret_cast<u128*>(d) = lo;
      *reinterpret_cast<u128*>(d + 16) = hi;
    }
  } else {  // 4 sums -> 8 bytes of a 16-bit type
    const uint64_t r = TO::pack(acc.f);
    uint8_t* d = out_base + o / 2;
    if (REMOTE) store64_relaxed_sys(d, r);
    else *reinterpret_cast<uint64_t*>(d) = r;
  }
}

static constexpr int kDirectUnroll = 4;

// Alignment of the boundaries between the slices of different CTAs.
static constexpr uint64_t kSplitAlignDirect = 128;

// Every rank's input and output as addresses valid on this rank (filled by the entry barrier).
struct PeerBufs {
  const uint8_t* const* in;
  uint8_t* const* out;
};

// out[i] = sum over ranks of in_q[i] for message bytes [byte_lo, byte_hi); the result is stored to
// `local_out` and, if PUSH, to the same offset of every peer's output.  Input offset o of the message lands
// at local_out + out_off(o - local_base).  FIXED_ORDER sums ranks 0..n-1 in that order on every rank (bitwise
// identical results everywhere, needed when several ranks reduce the same element); otherwise each rank
// starts at itself so that the n readers spread over the n memories.
template <class TI, class TO, int NTHREADS, bool PUSH, bool FIXED_ORDER, int NR, bool SLIM = false>
__device__ __forceinline__ void pull_reduce_range_n(const MtDevComm& c, const PeerBufs& P, uint8_t* local_out,
                                                    uint64_t byte_lo, uint64_t byte_hi, uint64_t local_base,
                                                    int nsrc = 0) {
  using CI = CastInfo<TI, TO>;
  // NR > 0: the number of sources is a compile-time constant, so the loop over them unrolls and all
  // NR x kU remote loads of a thread are in flight together.  NR == 0: `nsrc` sources (all ranks if 0).
  const int n = NR > 0 ? NR : (nsrc > 0 ? nsrc : c.nranks);
  // vectors per thread and pass: bounded so that NR x kU 16-byte registers fit without spilling
  // SLIM: half of that, for callers that keep more state alive around the call (chunk loops with counters);
  // with n - 1 remote sources a CTA still has tens of KiB in flight
  constexpr int kU = SLIM ? (NR >= 6 ? 1 : 2) : (NR >= 6 ? 2 : kDirectUnroll);
  // 16-byte vectors need every address involved to be aligned
  uint64_t mis = (uint64_t)(uintptr_t)(local_out + CI::out_off(byte_lo - local_base)) & CI::kOutAlignMask;
  for (int p = 0; p < n; ++p) {
    mis |= (uint64_t)(uintptr_t)(P.in[p] + byte_lo) & 15;
    if (PUSH && p != c.rank) mis |= (uint64_t)(uintptr_t)(P.out[p] + CI::out_off(byte_lo)) & CI::kOutAlignMask;
  }
  const uint64_t nvec = mis == 0 ? (byte_hi - byte_lo) >> 4 : 0;
  for (uint64_t base = 0; base < nvec; base += (uint64_t)NTHREADS * kU) {
    Acc128<TI> acc[kU];
    if (NR > 0) {
      u128 v[NR > 0 ? NR : 1][kU];
#pragma unroll
      for (int d = 0; d < NR; ++d) {
        const int p = FIXED_ORDER ? d : (c.rank + d) % NR;
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
          if (i < nvec) v[d][u] = load128_relaxed_sys(P.in[p] + byte_lo + (i << 4));
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
          if (i < nvec) v[u] = load128_relaxed_sys(P.in[p] + byte_lo + (i << 4));
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
        const uint64_t o = byte_lo + (i << 4);
        store_acc<TI, TO, false>(local_out, o - local_base, acc[u]);
        if (PUSH) {
          for (int d = 1; d < n; ++d) store_acc<TI, TO, true>(P.out[(c.rank + d) % n], o, acc[u]);
        }
      }
    }
  }
  // what the vectors did not cover (a tail of < 16 bytes, or everything when unaligned), element-wise
  using EI = typename TI::elem;
  using EO = typename TO::elem;
  const uint64_t done = byte_lo + (nvec << 4);
  const uint64_t nel = (byte_hi - done) / sizeof(EI);
  for (uint64_t e_i = threadIdx.x; e_i < nel; e_i += NTHREADS) {
    const uint64_t o = done + e_i * sizeof(EI);
    float acc = 0.f;
    for (int d = 0; d < n; ++d) {
      const int p = FIXED_ORDER ? d : (c.rank + d) % n;
      const EI x = *reinterpret_cast<const volatile EI*>(P.in[p] + o);
      acc += elem_to_float<TI>(x);
    }
    const EO e = float_to_elem<TO>(acc);
    *reinterpret_cast<EO*>(local_out + CI::out_off(o - local_base)) = e;
    if (PUSH)
      for (int d = 1; d < n; ++d) *reinterpret_cast<volatile EO*>(P.out[(c.rank + d) % n] + CI::out_off(o)) = e;
  }
}

template <class TI, class TO, int NTHREADS, bool PUSH, bool FIXED_ORDER, bool SLIM = false>
__device__ __forceinline__ void pull_reduce_range(const MtDevComm& c, const PeerBufs& P, uint8_t* local_out,
                                                  uint64_t byte_lo, uint64_t byte_hi, uint64_t local_base) {
  switch (c.nranks) {
    case 2: pull_reduce_range_n<TI, TO, NTHREADS, PUSH, FIXED_ORDER, 2, SLIM>(c, P, local_out, byte_lo, byte_hi, local_base); break;
    case 4: pull_reduce_range_n<TI, TO, NTHREADS, PUSH, FIXED_ORDER, 4, SLIM>(c, P, local_out, byte_lo, byte_hi, local_base); break;
    case 8: pull_reduce_range_n<TI, TO, NTHREADS, PUSH, FIXED_ORDER, 8, SLIM>(c, P, local_out, byte_lo, byte_hi, local_base); break;
    default: pull_reduce_range_n<TI, TO, NTHREADS, PUSH, FIXED_ORDER, 0, SLIM>(c, P, local_out, byte_lo, byte_hi, local_base); break;
  }
}

// Sum of `ns` sources (P.in[0 .. ns), in that order) over message bytes [byte_lo, byte_hi), stored at the same
// offsets of `dst` (local or a peer's memory).
template <class TI, class TO, int NTHREADS, int NR>
__device__ __forceinline__ void pull_reduce_sources_n(const MtDevComm& c, const PeerBufs& P, int ns, uint8_t* dst,
                                                      uint64_t byte_lo, uint64_t byte_hi) {
  pull_reduce_range_n<TI, TO, NTHREADS, false, true, NR, true>(c, P, dst, byte_lo, byte_hi, 0, ns);
}
template <class TI, class TO, int NTHREADS>
__device__ __forceinline__ void pull_reduce_sources(const MtDevComm& c, const PeerBufs& P, int ns, uint8_t* dst,
                                                    uint64_t byte_lo, uint64_t byte_hi) {
  switch (ns) {
    case 3: pull_reduce_sources_n<TI, TO, NTHREADS, 3>(c, P, ns, dst, byte_lo, byte_hi); break;
    case 7: pull_reduce_sources_n<TI, TO, NTHREADS, 7>(c, P, ns, dst, byte_lo, byte_hi); break;
    default: pull_reduce_sources_n<TI, TO, NTHREADS, 0>(c, P, ns, dst, byte_lo, byte_hi); break;
  }
}

// dst[i] = round(dst[i] + src[i]) over nbytes (a multiple of 16; both addresses 16-byte aligned).  dst was
// written by peers during this kernel, so it is read with system-scope loads.
template <class T, int NTHREADS>
__device__ __forceinline__ void add_into_range(uint8_t* dst, const uint8_t* src, uint64_t nbytes) {
  const uint64_t nvec = nbytes >> 4;
  for (uint64_t base = 0; base < nvec; base += (uint64_t)NTHREADS * kDirectUnroll) {
    u128 a[kDirectUnroll], b[kDirectUnroll];
#pragma unroll
    for (int u = 0; u < kDirectUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) {
        a[u] = load128_relaxed_sys(dst + (i << 4));
        b[u] = load128_stream(src + (i << 4));
      }
    }
#pragma unroll
    for (int u = 0; u < kDirectUnroll; ++u) {
      const uint64_t i = base + (uint64_t)u * NTHREADS + threadIdx.x;
      if (i < nvec) {
        Acc128<T> acc;
        acc.set(a[u]);
        acc.add(b[u]);
        *reinterpret_cast<u128*>(dst + (i << 4)) = acc.get();
      }
    }
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
// dst[i] = sum over all ranks of mc_src[i]; dst is local or peer memory, or the multicast alias when TO_MC.
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

// Bytes [lo, lo + nbytes) of every peer's output (but skip_rank's; and of the local one unless skip_local) = src,
// reading each vector once.  Any alignment: 16-byte vectors when src and every destination allow it, bytes otherwise
// and for the tail.
template <int NTHREADS>
__device__ __forceinline__ void bcast_fanout(const MtDevComm& c, const uint8_t* src, const PeerBufs& P, uint64_t lo,
                                             uint64_t nbytes, bool skip_local, int skip_rank = -1) {
  const int n = c.nranks;
  uint64_t mis = (uint64_t)(uintptr_t)src & 15;
  for (int p = 0; p < n; ++p) mis |= (uint64_t)(uintptr_t)(P.out[p] + lo) & 15;
  const uint64_t nvec = mis == 0 ? nbytes >> 4 : 0;
  uint8_t* local_dst = P.out[c.rank] + lo;
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
        for (int d = 1; d < n; ++d) {
          const int p = (c.rank + d) % n;
          if (p != skip_rank) store128_relaxed_sys(P.out[p] + lo + (i << 4), v[u]);
        }
        if (!skip_local) *reinterpret_cast<u128*>(local_dst + (i << 4)) = v[u];
      }
    }
  }
  for (uint64_t o = (nvec << 4) + threadIdx.x; o < nbytes; o += NTHREADS) {
    const uint8_t b = *reinterpret_cast<const volatile uint8_t*>(src + o);
    for (int d = 1; d < n; ++d) {
      const int p = (c.rank + d) % n;
      if (p != skip_rank) *reinterpret_cast<volatile uint8_t*>(P.out[p] + lo + o) = b;
    }
    if (!skip_local) local_dst[o] = b;
  }
}

// ---- copy-engine variants ---------------------------------------------------------------------------
// One thread per CTA drives bulk copies (cp.async.bulk): a piece of the source is fetched into a ring of
// shared-memory slots and stored from there to every destination, so that each byte is read from HBM (or
// pulled over NVLink) once however many peers receive it, a CTA keeps up to kBulkSlots x kBulkPiece bytes in
// flight without holding them in registers, and a few tens of CTAs saturate the link.  Loads run kBulkLag
// pieces ahead of the stores.  Nothing here replicates a load across a cluster; the only multi-destination
// operation is the loop over peers issuing one store each.  Every wait is bounded.
constexpr uint32_t kBulkPiece = 32768;
constexpr int kBulkSlots = 6, kBulkLag = 3;
constexpr uint32_t kBulkSmemBytes = kBulkSlots * kBulkPiece + 1024;   // + room to align the ring to 1024 bytes

struct BulkJob {
  const uint8_t* src;
  uint64_t nbytes;                 // multiple of 16
  int32_t ndst;
  uint8_t* dst[MT_MAX_RANKS];
};
struct BulkCtl {
  uint64_t full[kBulkSlots];
  int abort;
  int njobs;
  BulkJob jobs[MT_MAX_RANKS];
};

__device__ __forceinline__ bool bulk_mbar_wait(uint64_t* bar, uint32_t parity, uint64_t timeout_ns) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!tc::mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ffu) == 0) {
      const uint64_t now = globaltimer();
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) return false;
    }
  }
  return true;
}

// Runs the jobs of ctl (thread 0 of the CTA only).  Returns false if a load never completed.
static __device__ bool bulk_run(BulkCtl* ctl, uint8_t* ring, uint64_t timeout_ns) {
  using namespace tc;
  for (int s = 0; s < kBulkSlots; ++s) mbar_init(&ctl->full[s], 1);
  fence_barrier_init();
  uint32_t total = 0;
  for (int j = 0; j < ctl->njobs; ++j) total += (uint32_t)mt_div_up(ctl->jobs[j].nbytes, kBulkPiece);
  // two cursors over (job, piece): `l` for loads, `t` for stores
  int lj = 0, tj = 0;
  uint64_t lo = 0, to = 0;
  bool ok = true;
  for (uint32_t i = 0; ok && i < total + kBulkLag; ++i) {
    if (i < total) {
      while (lo >= ctl->jobs[lj].nbytes) {
        ++lj;
        lo = 0;
      }
      const BulkJob& J = ctl->jobs[lj];
      const uint64_t left = J.nbytes - lo;
      const uint32_t nb = (uint32_t)(left < kBulkPiece ? left : kBulkPiece);
      const uint32_t slot = i % kBulkSlots;
      // the stores that last used this slot (piece i - kBulkSlots) must have finished reading it
      if (i >= kBulkSlots) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kBulkSlots - kBulkLag - 1) : "memory");
      mbar_expect_tx(&ctl->full[slot], nb);
      bulk_load_1d(ring + (uint64_t)slot * kBulkPiece, J.src + lo, nb, &ctl->full[slot]);
      lo += nb;
    }
    if (i >= kBulkLag) {
      const uint32_t k = i - kBulkLag;
      while (to >= ctl->jobs[tj].nbytes) {
        ++tj;
        to = 0;
      }
      const BulkJob& J = ctl->jobs[tj];
      const uint64_t left = J.nbytes - to;
      const uint32_t nb = (uint32_t)(left < kBulkPiece ? left : kBulkPiece);
      const uint32_t slot = k % kBulkSlots;
      if (!bulk_mbar_wait(&ctl->full[slot], (k / kBulkSlots) & 1, timeout_ns)) {
        ok = false;
        break;
      }
      for (int d = 0; d < J.ndst; ++d)
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(J.dst[d] + to),
                     "r"(smem_u32(ring + (uint64_t)slot * kBulkPiece)), "r"(nb)
                     : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      to += nb;
    }
  }
  // every store has completed (not merely left shared memory) before the CTA goes on to the exit barrier,
  // whose release publishes them
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  return ok;
}

// Are all the addresses of the jobs multiples of 16?  (Sizes are cut to multiples of 16 by the caller.)
__device__ __forceinline__ bool bulk_aligned(const BulkCtl* ctl) {
  uint64_t mis = 0;
  for (int j = 0; j < ctl->njobs; ++j) {
    mis |= (uint64_t)(uintptr_t)ctl->jobs[j].src;
    for (int d = 0; d < ctl->jobs[j].ndst; ++d) mis |= (uint64_t)(uintptr_t)ctl->jobs[j].dst[d];
  }
  return (mis & 15) == 0;
}

// The n - 1 other ranks each sum one sub-slice of THEIR OWN inputs (the root's is left out) and store the
// partial result into the root's output, chunk by chunk, raising a counter in the root's barrier slot
// after each chunk; the root adds its own input to every chunk as it arrives.  Nobody reads the root's
// memory.  Measured reason (4 B200, 256 MiB): with the root as one of the read sources (variant 3) the
// call takes 568 us, without it 433 us, without the stores into the root 414 us.  The stores (write
// requests carrying data) fill the root's incoming link, and read requests to the root wait behind them.
// The price is a second rounding (the partial sum is rounded into the output type before the root adds)
// and the root's own pass over the output: measured 500 us for 256 MiB on 4 B200 (variant 3: 566, in-switch
// sum: 508) and 169 us for 64 MiB (165, 146); 482 / 159 us once the chunk loop stopped spilling registers.  The
// choice for large messages in memory the switch cannot sum.  (Tried and dropped: the others sum into staging
// slots of their own and the root pulls them, so that all bulk data travels as read responses.  730 us: a root
// CTA that pulls 64 KiB chunks from n - 1 producers in turn is bound by the latency of each chunk.)
template <class T, int NTHREADS>
__device__ __forceinline__ void reduce_summing_root(const MtDevComm& c, const DirectArgs& a, const PeerBufs& P,
                                                 const uint8_t* in, uint8_t* out, MtRange r, int cta, int* s_fail) {
  using TI = T;
  using TO = T;
  const int n = c.nranks, me = c.rank;
  constexpr uint64_t kChunk = 256u << 10;   // 64 KiB chunks cost 10 % (a fence and a counter per chunk), 512 KiB and up lengthen the root's tail
  __shared__ uint64_t s_tag;
  const uint64_t len = r.hi - r.lo;
  MtBarSlot* mine = (MtBarSlot*)(c.heap[me] + c.L.bar_off) + cta;
  // the slot's epoch moves in step on all ranks (every barrier on a slot includes every rank), so it
  // tags the counters of this call: older calls left smaller values
  if (threadIdx.x == 0) s_tag = load64(&mine->epoch) << 24;
  __syncthreads();
  const uint64_t tag = s_tag;
  if (me != a.root) {
    const int idx = mt_mod(me - a.root - 1, n);
    const MtRange sm = mt_split(len, n - 1, idx, 128);
    const uint8_t* src[MT_MAX_RANKS];
    int ns = 0;
    for (int d = 0; d < n; ++d) {   // this rank first, then the others in ring order, the root left out
      const int p = (me + d) % n;
      if (p != a.root) src[ns++] = P.in[p];
    }
    const PeerBufs Q{src, P.out};
    MtBarSlot* roots = (MtBarSlot*)(c.heap[a.root] + c.L.bar_off) + cta;
    uint64_t k = 0;
    for (uint64_t lo = sm.lo; lo < sm.hi; lo += kChunk, ++k) {
      const uint64_t hi = mt_min64(lo + kChunk, sm.hi);
      pull_reduce_sources<TI, TO, NTHREADS>(c, Q, ns, P.out[a.root], r.lo + lo, r.lo + hi);
      __syncthreads();
      if (threadIdx.x == 0) {
        fence_acq_rel_sys();   // the CTA's stores into the root have landed before the counter moves
        store64_release_sys(&roots->xflag[me], tag + k + 1);
      }
    }
  } else {
    uint64_t nchunks = 0;
    for (int j = 0; j < n - 1; ++j) {
      const MtRange sm = mt_split(len, n - 1, j, 128);
      const uint64_t nc = mt_div_up(sm.hi - sm.lo, kChunk);
      if (nc > nchunks) nchunks = nc;
    }
    bool ok = true;
    for (uint64_t k = 0; ok && k < nchunks; ++k) {
      for (int j = 0; ok && j < n - 1; ++j) {
        const int p = (a.root + 1 + j) % n;   // the rank with sub-slice j
        const MtRange sm = mt_split(len, n - 1, j, 128);
        const uint64_t lo = sm.lo + k * kChunk;
        if (lo >= sm.hi) continue;
        const uint64_t hi = mt_min64(lo + kChunk, sm.hi);
        if (threadIdx.x == 0) {
          const uint64_t want = tag + k + 1;
          const uint64_t* w = &mine->xflag[p];
          if (!bounded_wait(
                  c, [&] { return load64_acquire_sys(w) >= want; }, MT_ERR_TIMEOUT_FLAG, cta,
                  MT_WHERE_CHUNK_FLAG, want, k, (const volatile uint64_t*)w))
            atomicExch(s_fail, 1);
        }
        __syncthreads();
        ok = *s_fail == 0;
        if (ok) add_into_range<TI, NTHREADS>(out + r.lo + lo, in + r.lo + lo, hi - lo);
      }
    }
  }
}

template <class TI, class TO, int NTHREADS>
__device__ void direct_body(const MtDevComm& c, const DirectArgs& a, int lr, int cta, int ncta, int* s_fail,
                            const uint8_t** s_in, uint8_t** s_out, BulkCtl* ctl, uint8_t* ring) {
  using T = TI;
  constexpr bool kSame = CastInfo<TI, TO>::kSame;
  const int n = c.nranks, me = c.rank;
  const uint8_t* in = (const uint8_t*)a.in[lr];
  uint8_t* out = (uint8_t*)a.out[lr];
  const uint64_t B = a.nbytes;

  {
    const int t = threadIdx.x & (MT_MAX_RANKS - 1);
    const uint64_t vin = a.pub_local ? (uint64_t)(uintptr_t)in : a.pub_in[t];
    const uint64_t vout = a.pub_local ? (uint64_t)(uintptr_t)out : a.pub_out[t];
    if (!rank_barrier_xchg(c, cta, s_fail, vin, vout, in, out, s_in, s_out)) return;
  }
  const PeerBufs P{s_in, s_out};

  switch (a.op) {
    case DOP_ALLGATHER: {
      if constexpr (kSame) {
        const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
        if (r.hi > r.lo) {
          if (a.nvls) {
            // one multimem store lands in every rank's output (mine included)
            uint8_t* mdst = c.mc + a.mc_out_off + (uint64_t)me * B;
            const uint64_t nvec = (r.hi - r.lo) >> 4;
            nvls_bcast_range<NTHREADS>(in + r.lo, mdst + r.lo, nvec);
            // a tail cannot be sent with 16-byte multimem stores
            for (uint64_t o = r.lo + (nvec << 4) + threadIdx.x; o < r.hi; o += NTHREADS)
              for (int p = 0; p < n; ++p) *(volatile uint8_t*)(P.out[p] + (uint64_t)me * B + o) = in[o];
          } else if (a.variant == 0 || a.variant == 4) {
            bool done = false;
            if (a.variant == 4) {
              // copy engine: each piece of my shard is read once and stored to every rank from shared memory
              if (threadIdx.x == 0) {
                BulkJob& J = ctl->jobs[0];
                J.src = in + r.lo;
                J.nbytes = (r.hi - r.lo) & ~15ull;
                J.ndst = 0;
                for (int d = 1; d <= n; ++d) {   // the peers first, my own copy last
                  const int p = (me + d) % n;
                  uint8_t* dst = P.out[p] + (uint64_t)me * B;
                  if (p == me && in == dst) continue;
                  J.dst[J.ndst++] = dst + r.lo;
                }
                ctl->njobs = 1;
                ctl->abort = bulk_aligned(ctl) ? 0 : 2;   // 2: not aligned, the threads copy instead
                if (ctl->abort == 0 && !bulk_run(ctl, ring, c.timeout_ns)) {
                  ctl->abort = 1;
                  report_error(c, MT_ERR_TIMEOUT_FLAG, cta, MT_WHERE_BULK, 0, 0, 0);
                }
              }
              __syncthreads();
              done = ctl->abort != 2;
              if (done && ctl->abort == 0) {   // the last < 16 bytes
                for (uint64_t o = r.lo + ((r.hi - r.lo) & ~15ull) + threadIdx.x; o < r.hi; o += NTHREADS)
                  for (int p = 0; p < n; ++p) {
                    uint8_t* dst = P.out[p] + (uint64_t)me * B;
                    if (!(p == me && in == dst)) *(volatile uint8_t*)(dst + o) = in[o];
                  }
              }
            }
            if (!done) {
              for (int d = 0; d < n; ++d) {
                const int p = (me + d) % n;
                uint8_t* dst = P.out[p] + (uint64_t)me * B;
                if (p == me && in == dst) continue;
                copy_range<NTHREADS, false, true>(in + r.lo, dst + r.lo, r.hi - r.lo);
              }
            }
          } else {
            bool done = false;
            if (a.variant == 5) {
              // copy engine, pulling: one stream per peer from its contribution into my output
              if (threadIdx.x == 0) {
                int nj = 0;
                for (int d = 1; d <= n; ++d) {   // the peers first, my own copy last
                  const int p = (me + d) % n;
                  const uint8_t* src = p == me ? in : P.in[p];
                  uint8_t* dst = out + (uint64_t)p * B;
                  if (p == me && in == dst) continue;
                  BulkJob& J = ctl->jobs[nj++];
                  J.src = src + r.lo;
                  J.nbytes = (r.hi - r.lo) & ~15ull;
                  J.ndst = 1;
                  J.dst[0] = dst + r.lo;
                }
                ctl->njobs = nj;
                ctl->abort = bulk_aligned(ctl) ? 0 : 2;
                if (ctl->abort == 0 && nj > 0 && !bulk_run(ctl, ring, c.timeout_ns)) {
                  ctl->abort = 1;
                  report_error(c, MT_ERR_TIMEOUT_FLAG, cta, MT_WHERE_BULK, 0, 0, 0);
                }
              }
              __syncthreads();
              done = ctl->abort != 2;
              if (done && ctl->abort == 0) {
                for (uint64_t o = r.lo + ((r.hi - r.lo) & ~15ull) + threadIdx.x; o < r.hi; o += NTHREADS)
                  for (int p = 0; p < n; ++p) {
                    const uint8_t* src = p == me ? in : P.in[p];
                    uint8_t* dst = out + (uint64_t)p * B;
                    if (!(p == me && in == dst)) dst[o] = *(const volatile uint8_t*)(src + o);
                  }
              }
            }
            for (int d = 0; !done && d < n; ++d) {
              const int p = (me + d) % n;
              if (p == me) {
                if (in != out + (uint64_t)me * B) copy_range<NTHREADS, false, false>(in + r.lo, out + (uint64_t)me * B + r.lo, r.hi - r.lo);
              } else {
                copy_range<NTHREADS, true, false>(P.in[p] + r.lo, out + (uint64_t)p * B + r.lo, r.hi - r.lo);
              }
            }
          }
        }
      }
      break;
    }
    case DOP_ALLTOALL: {
      if constexpr (kSame) {
        const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
        bool done = false;
        if (r.hi > r.lo && a.variant == 4) {
          // copy engine: one stream per peer, block p of my input into slot `me` of p's output
          if (threadIdx.x == 0) {
            for (int d = 0; d < n; ++d) {
              const int p = (me + 1 + d) % n;
              BulkJob& J = ctl->jobs[d];
              J.src = in + (uint64_t)p * B + r.lo;
              J.nbytes = (r.hi - r.lo) & ~15ull;
              J.ndst = 1;
              J.dst[0] = P.out[p] + (uint64_t)me * B + r.lo;
            }
            ctl->njobs = n;
            ctl->abort = bulk_aligned(ctl) ? 0 : 2;
            if (ctl->abort == 0 && !bulk_run(ctl, ring, c.timeout_ns)) {
              ctl->abort = 1;
              report_error(c, MT_ERR_TIMEOUT_FLAG, cta, MT_WHERE_BULK, 0, 0, 0);
            }
          }
          __syncthreads();
          done = ctl->abort != 2;
          if (done && ctl->abort == 0) {
            for (uint64_t o = r.lo + ((r.hi - r.lo) & ~15ull) + threadIdx.x; o < r.hi; o += NTHREADS)
              for (int p = 0; p < n; ++p) *(volatile uint8_t*)(P.out[p] + (uint64_t)me * B + o) = in[(uint64_t)p * B + o];
          }
        }
        if (r.hi > r.lo && !done) {
          for (int d = 0; d < n; ++d) {
            const int p = (me + d) % n;
            if (a.variant == 0 || a.variant == 4) {  // push block p of my input into slot `me` of p's output
              uint8_t* dst = P.out[p] + (uint64_t)me * B;
              copy_range<NTHREADS, false, true>(in + (uint64_t)p * B + r.lo, dst + r.lo, r.hi - r.lo);
            } else {  // pull block `me` of p's input into slot p of my output
              const uint8_t* src = P.in[p] + (uint64_t)me * B;
              copy_range<NTHREADS, true, false>(src + r.lo, out + (uint64_t)p * B + r.lo, r.hi - r.lo);
            }
          }
        }
      }
      break;
    }
    case DOP_REDUCESCATTER: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (r.hi > r.lo) {
        const uint64_t so = (uint64_t)me * B;
        if (kSame && a.nvls) {
          if constexpr (kSame) {
            const uint8_t* msrc = c.mc + a.mc_in_off + so;
            const uint64_t nvec = (r.hi - r.lo) >> 4;
            nvls_reduce_range<T, NTHREADS, false>(msrc + r.lo, out + r.lo, nvec);
            if (r.lo + (nvec << 4) < r.hi)
              pull_reduce_range<TI, TO, NTHREADS, false, false>(c, P, out, so + r.lo + (nvec << 4), so + r.hi, so);
          }
        } else {
          pull_reduce_range<TI, TO, NTHREADS, false, false>(c, P, out, so + r.lo, so + r.hi, so);
        }
      }
      break;
    }
    case DOP_ALLREDUCE: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (r.hi > r.lo) {
        if (a.variant == 1) {  // one-shot: everybody sums everything, writes locally only
          pull_reduce_range<TI, TO, NTHREADS, false, true>(c, P, out, r.lo, r.hi, 0);
        } else {
          // two-shot: inside this CTA's slice, rank `me` owns sub-slice `me`
          const MtRange s = mt_split(r.hi - r.lo, n, me, 16);
          const uint64_t lo = r.lo + s.lo, hi = r.lo + s.hi;
          if (hi > lo) {
            if (kSame && a.nvls) {
              if constexpr (kSame) {
                const uint64_t nvec = (hi - lo) >> 4;
                nvls_reduce_range<T, NTHREADS, true>(c.mc + a.mc_in_off + lo, c.mc + a.mc_out_off + lo, nvec);
                if (lo + (nvec << 4) < hi)
                  pull_reduce_range<TI, TO, NTHREADS, true, false>(c, P, out, lo + (nvec << 4), hi, 0);
              }
            } else {
              pull_reduce_range<TI, TO, NTHREADS, true, false>(c, P, out, lo, hi, 0);
            }
          }
        }
      }
      break;
    }
    case DOP_BROADCAST: {
      if constexpr (kSame) {
        const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
        if (a.variant == 2 || a.variant == 4) {
          // pull + replicate: a rank fetches one sub-slice straight from the root's buffer and replicates it
          // (one multimem.st per vector, or plain / bulk stores to every peer).  The root's link carries each
          // byte once, the replication is spread over the ranks (a single source of multicast stores tops out
          // near 400 GB/s), and there is no phase in which only the root's link is busy.  With multicast
          // stores all n ranks take a sub-slice (the root's copy leaves its link once).  With plain stores
          // only the n - 1 other ranks do: a root that also replicated a sub-slice to n - 1 peers would put
          // 2 (n - 1) / n message sizes on its outgoing link, where every other link carries one.
          const uint64_t len = r.hi - r.lo;
          const bool others_only = !a.nvls && n > 2;
          const int nsl = others_only ? n - 1 : n;
          const int idx = others_only ? mt_mod(me - a.root - 1, n) : me;   // the root: n - 1, no sub-slice
          const int skip_rank = others_only ? a.root : -1;
          if (others_only && me == a.root) {
            if (in != out && len) copy_range<NTHREADS, false, false>(in + r.lo, out + r.lo, len);
            break;
          }
          // n - 1 sub-slices do not fall on 128-byte lines by themselves (n sub-slices of a 128-aligned range do
          // for a power-of-two n): ask for it, so that warps and bulk copies move whole lines
          const MtRange sm = mt_split(len, nsl, idx, others_only ? 128 : 16);
          if (sm.hi > sm.lo) {
            const uint8_t* src = (me == a.root ? in : P.in[a.root]) + r.lo + sm.lo;
            const uint64_t nb = sm.hi - sm.lo;
            if (a.nvls) {
              if (me == a.root) nvls_bcast_range<NTHREADS, false>(src, c.mc + a.mc_out_off + r.lo + sm.lo, nb >> 4);
              else nvls_bcast_range<NTHREADS, true>(src, c.mc + a.mc_out_off + r.lo + sm.lo, nb >> 4);
            } else {
              bool done = false;
              const bool skip_self = me == a.root && in == out;
              if (a.variant == 4) {
                // copy engine: the sub-slice crosses the root's link once (a bulk load from the root's memory)
                // and is stored to every rank from shared memory
                if (threadIdx.x == 0) {
                  BulkJob& J = ctl->jobs[0];
                  J.src = src;
                  J.nbytes = nb & ~15ull;
                  J.ndst = 0;
                  for (int d = 1; d <= n; ++d) {
                    const int p = (me + d) % n;
                    if ((p == me && skip_self) || p == skip_rank) continue;
                    J.dst[J.ndst++] = P.out[p] + r.lo + sm.lo;
                  }
                  ctl->njobs = 1;
                  ctl->abort = bulk_aligned(ctl) ? 0 : 2;
                  if (ctl->abort == 0 && !bulk_run(ctl, ring, c.timeout_ns)) {
                    ctl->abort = 1;
                    report_error(c, MT_ERR_TIMEOUT_FLAG, cta, MT_WHERE_BULK, 0, 0, 0);
                  }
                }
                __syncthreads();
                done = ctl->abort != 2;
                if (done && ctl->abort == 0 && (nb & 15))
                  bcast_fanout<NTHREADS>(c, src + (nb & ~15ull), P, r.lo + sm.lo + (nb & ~15ull), nb & 15, skip_self, skip_rank);
              }
              if (!done) bcast_fanout<NTHREADS>(c, src, P, r.lo + sm.lo, nb, skip_self, skip_rank);
            }
          }
          break;
        }
        if (r.hi > r.lo) {
          if (a.nvls) {
            if (me == a.root) {
              const uint64_t nvec = (r.hi - r.lo) >> 4;
              nvls_bcast_range<NTHREADS>(in + r.lo, c.mc + a.mc_out_off + r.lo, nvec);
              for (uint64_t o = r.lo + (nvec << 4) + threadIdx.x; o < r.hi; o += NTHREADS)
                for (int p = 0; p < n; ++p) *(volatile uint8_t*)(P.out[p] + o) = in[o];
            }
          } else if (a.variant == 0) {
            if (me == a.root) {
              for (int d = 0; d < n; ++d) {
                const int p = (me + d) % n;
                if (p == me && in == out) continue;
                copy_range<NTHREADS, false, true>(in + r.lo, P.out[p] + r.lo, r.hi - r.lo);
              }
            }
          } else {
            if (me != a.root) copy_range<NTHREADS, true, false>(P.in[a.root] + r.lo, out + r.lo, r.hi - r.lo);
            else if (in != out) copy_range<NTHREADS, false, false>(in + r.lo, out + r.lo, r.hi - r.lo);
          }
        }
      }
      break;
    }
    case DOP_REDUCE: {
      const MtRange r = mt_split(B, ncta, cta, kSplitAlignDirect);
      if (a.variant == 2) {
        // reduce-scatter + gather: rank j sums sub-slice j in the switch and stores the result straight into
        // the root's output, so the summing is spread over all ranks and the root only receives.
        if constexpr (kSame) {
          const MtRange sm = mt_split(r.hi - r.lo, n, me, 16);
          if (sm.hi > sm.lo) {
            const uint64_t lo = r.lo + sm.lo, hi = r.lo + sm.hi;
            uint8_t* dst = P.out[a.root];
            if (a.nvls) {
              nvls_reduce_range<T, NTHREADS, false>(c.mc + a.mc_in_off + lo, dst + lo, (hi - lo) >> 4);
            } else {
              pull_reduce_range<TI, TO, NTHREADS, false, false>(c, P, dst, lo, hi, 0);
            }
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
          const MtRange sm = mt_split(r.hi - r.lo, n - 1, idx, 128);   // whole 128-byte lines per warp
          if (sm.hi > sm.lo)
            pull_reduce_range<TI, TO, NTHREADS, false, false>(c, P, P.out[a.root], r.lo + sm.lo, r.lo + sm.hi, 0);
        }
        break;
      }
      if (r.hi > r.lo && me == a.root) {
        if (kSame && a.nvls) {
          if constexpr (kSame) {
            const uint64_t nvec = (r.hi - r.lo) >> 4;
            nvls_reduce_range<T, NTHREADS, false>(c.mc + a.mc_in_off + r.lo, out + r.lo, nvec);
            if (r.lo + (nvec << 4) < r.hi)
              pull_reduce_range<TI, TO, NTHREADS, false, false>(c, P, out, r.lo + (nvec << 4), r.hi, 0);
          }
        } else {
          pull_reduce_range<TI, TO, NTHREADS, false, false>(c, P, out, r.lo, r.hi, 0);
        }
      }
      break;
    }
    default: break;
  }

  rank_barrier(c, cta, s_fail);
}

template <class TI, class TO, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS, 1) direct_kernel(const MtDevComm* comms, DirectArgs a) {
  extern __shared__ uint8_t dyn_smem[];   // kBulkSmemBytes for the copy-engine variants, else nothing
  __shared__ int s_fail;
  __shared__ const uint8_t* s_in[MT_MAX_RANKS];
  __shared__ uint8_t* s_out[MT_MAX_RANKS];
  __shared__ BulkCtl ctl;
  const int lr = blockIdx.y;
  uint8_t* ring = (uint8_t*)(((uintptr_t)dyn_smem + 1023) & ~(uintptr_t)1023);
  direct_body<TI, TO, NTHREADS>(comms[lr], a, lr, blockIdx.x, gridDim.x, &s_fail, s_in, s_out, &ctl, ring);
}

// The reduce variant with per-chunk counters between the other ranks and the root (variant 5: summing root), as a
// kernel of its own: its registers are allocated apart from direct_kernel's.
template <class T, int NTHREADS>
__global__ void __launch_bounds__(NTHREADS, 1) rooted_reduce_kernel(const MtDevComm* comms, DirectArgs a) {
  __shared__ int s_fail;
  __shared__ const uint8_t* s_in[MT_MAX_RANKS];
  __shared__ uint8_t* s_out[MT_MAX_RANKS];
  const int lr = blockIdx.y, cta = blockIdx.x;
  const MtDevComm& c = comms[lr];
  const uint8_t* in = (const uint8_t*)a.in[lr];
  uint8_t* out = (uint8_t*)a.out[lr];
  {
    const int t = threadIdx.x & (MT_MAX_RANKS - 1);
    const uint64_t vin = a.pub_local ? (uint64_t)(uintptr_t)in : a.pub_in[t];
    const uint64_t vout = a.pub_local ? (uint64_t)(uintptr_t)out : a.pub_out[t];
    if (!rank_barrier_xchg(c, cta, &s_fail, vin, vout, in, out, s_in, s_out)) return;
  }
  const PeerBufs P{s_in, s_out};
  const MtRange r = mt_split(a.nbytes, gridDim.x, cta, kSplitAlignDirect);
  reduce_summing_root<T, NTHREADS>(c, a, P, in, out, r, cta, &s_fail);
  rank_barrier(c, cta, &s_fail);
}

}  // namespace mt
