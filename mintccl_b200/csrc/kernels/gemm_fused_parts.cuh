// Parts shared by the GEMM kernels that are fused with a collective (gemm_tc.cu: single-CTA tiles, gemm_tc2.cu:
// CTA pairs): bounded mbarrier wait, error report, the comm CTAs of all-gather -> GEMM and the reducer of
// GEMM -> reduce-scatter.  The layouts they share with the GEMM CTAs:
//   all-gather -> GEMM      gathered A [M, K] at heap offset gather_off; one arrival counter per (source rank,
//                           128-row block) at flags_off, counted once per call by every comm CTA of a group
//   GEMM -> reduce-scatter  partial tiles, tile-major [source rank][128-row block][256-col block][128 x 256]
//                           bf16 at stage_off on the owner of the rows; one counter per partial tile at
//                           flags_off, counted by the 4 epilogue warps that wrote it; two ticket words behind
//
// The reference has no compute kernels (README.md:5 only asks that collectives fuse with others).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../device/prims.cuh"
#include "../device/sched.h"
#include "../device/tc_prims.cuh"
#include "gemm_tc.h"

namespace mt {
namespace fused {
using namespace tc;

constexpr int BM = 128, BN = 256;   // rows of a row block / arrival counter, columns of a tile
constexpr int kGemmThreads = 192;   // threads of every CTA of the fused kernels

// comm CTAs: ring of COMM_SLOTS pieces in shared memory, loads run COMM_LAG pieces ahead of stores
constexpr uint32_t COMM_PIECE = 32768;
constexpr int COMM_SLOTS = 6, COMM_LAG = 3, COMM_SIGLAG = 12;
struct CommCtl {
  uint64_t full[COMM_SLOTS];
  int abort;
};

// Bounded mbarrier wait.  Returns false after the time limit or when the CTA-wide abort flag is up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint64_t timeout_ns) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ffu) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer();
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void gemm_report(const GemmArgs& a, int lr, uint32_t where) {
  if (a.status[lr]) {
    MtStatus* st = (MtStatus*)a.status[lr];
    if (atomicCAS(&st->code, 0u, (uint32_t)MT_ERR_TIMEOUT_FLAG) == 0u) {
      st->rank = a.rank[lr];
      st->channel = blockIdx.x;
      st->where = where;
    }
    store32_relaxed_sys(&st->abort, 1u);
  }
}

// Reducer of GEMM -> reduce-scatter: output tiles of this rank are handed out by tickets (an atomic
// counter that alternates between two words from call to call; the idle one is zeroed for the next
// call), in the order in which their partial tiles complete.  A CTA takes tickets until none is left.
static __device__ void rs_reduce_loop(const GemmArgs& a, int lr) {
  const MtDevComm& c = a.comms[lr];
  const int n = a.nranks, me = a.rank[lr];
  const int per_rows = a.M / n, per = per_rows / BM, nbs = a.N / BN;
  const uint64_t ld_bytes = (uint64_t)a.N * 2;
  const uint8_t* stage = c.heap[me] + a.stage_off;
  uint64_t* cnts = (uint64_t*)(c.heap[me] + a.flags_off);
  unsigned long long* tickets = (unsigned long long*)(cnts + (uint64_t)n * per * nbs);
  const uint64_t timeout_ns = a.timeout_ns;
  __shared__ int s_ok, s_ot;
  if (blockIdx.x == 0 && threadIdx.x == 0) tickets[(a.epoch + 1) & 1] = 0;  // next call's counter
  while (true) {
    __syncthreads();
    if (threadIdx.x == 0) {
      s_ok = 1;
      s_ot = (int)atomicAdd(&tickets[a.epoch & 1], 1ull);
      if (s_ot < per * nbs) {
        const int mbl = s_ot / nbs, nb = s_ot % nbs;
        const uint64_t want = a.epoch * 4ull;  // four epilogue warps count each partial tile
        for (int s = 0; s < n && s_ok; ++s) {
          const uint64_t* w = cnts + ((uint64_t)s * per + mbl) * nbs + nb;
          uint32_t spins = 0;
          uint64_t t0 = 0;
          while (load64_acquire_sys(w) < want) {
            if ((++spins & 0xffu) == 0) {
              const uint64_t now = globaltimer();
              if (t0 == 0) t0 = now;
              else if (now - t0 > timeout_ns) {
                s_ok = 0;
                gemm_report(a, lr, MT_WHERE_GEMM_FLAG);
                break;
              }
            }
            __nanosleep(40);
          }
        }
      }
    }
    __syncthreads();
    const int ot = s_ot;
    if (!s_ok || ot >= per * nbs) return;
    {
      const int mbl = ot / nbs, nb = ot % nbs;
      // 128 x 256 bf16 output tile: 4096 vectors of 16 bytes (8 elements)
      uint8_t* out = (uint8_t*)a.c[lr] + (uint64_t)mbl * BM * ld_bytes + (uint64_t)nb * BN * 2;
      constexpr int RU = 4;  // vectors per thread and pass: RU x ranks loads in flight
      for (int v0 = threadIdx.x; v0 < BM * (BN / 8); v0 += kGemmThreads * RU) {
        float acc[RU][8];
#pragma unroll
        for (int u = 0; u < RU; ++u)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
        for (int s = 0; s < n; ++s) {
          u128 w[RU];
#pragma unroll
          for (int u = 0; u < RU; ++u) {
            const int v = v0 + u * kGemmThreads;
            if (v < BM * (BN / 8)) {
              const int rr = v / (BN / 8), cv = v % (BN / 8);
              w[u] = load128_relaxed_sys(stage + (((uint64_t)s * per + mbl) * nbs + nb) * (uint64_t)(BM * BN * 2) +
                                         (uint64_t)rr * (BN * 2) + cv * 16);
            }
          }
#pragma unroll
          for (int u = 0; u < RU; ++u) {
            const uint32_t ww[4] = {(uint32_t)w[u].x, (uint32_t)(w[u].x >> 32), (uint32_t)w[u].y, (uint32_t)(w[u].y >> 32)};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[u][2 * e] += __uint_as_float(ww[e] << 16);
              acc[u][2 * e + 1] += __uint_as_float(ww[e] & 0xffff0000u);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < RU; ++u) {
          const int v = v0 + u * kGemmThreads;
          if (v < BM * (BN / 8)) {
            const int rr = v / (BN / 8), cv = v % (BN / 8);
            uint4 o;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(acc[u][0], acc[u][1]), p1 = __floats2bfloat162_rn(acc[u][2], acc[u][3]);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(acc[u][4], acc[u][5]), p3 = __floats2bfloat162_rn(acc[u][6], acc[u][7]);
            o.x = *(uint32_t*)&p0; o.y = *(uint32_t*)&p1; o.z = *(uint32_t*)&p2; o.w = *(uint32_t*)&p3;
            *(uint4*)(out + (uint64_t)rr * ld_bytes + cv * 16) = o;
          }
        }
      }
    }
  }
}

// One comm CTA of the all-gather fusion: moves 128-row chunks of this rank's rows to the peers (push) or of the
// peers' rows to this rank (pull) while the other CTAs of the grid run the GEMM, and counts every chunk on the
// consumer's arrival counter.  `cc` is the index of this CTA among the `ncomm` comm CTAs, `smem` a
// 1024-byte-aligned area of COMM_SLOTS x COMM_PIECE bytes, `cm` a control block behind it.
template <bool FP8>
__device__ __forceinline__ void ag_comm_cta(const GemmArgs& a, int lr, int cc, int ncomm, uint8_t* smem, CommCtl* cm) {
  const MtDevComm& c = a.comms[lr];
  const uint64_t timeout_ns = a.timeout_ns;
  __shared__ int s_fail;
  // every rank has entered this call, so nobody still reads last call's gathered rows
  if (!rank_barrier(c, cc, &s_fail)) return;
  const int n = c.nranks, me = c.rank;
  const uint64_t row_bytes = (uint64_t)a.K * (FP8 ? 1 : 2);
  const uint64_t shard_rows = a.M / n;
  const int chunks = (int)(shard_rows / BM);
  const uint8_t* src = (const uint8_t*)a.a_local[lr];
  // One thread drives the copy engine: bulk copies local HBM -> shared memory ring -> peer HBM, so a
  // handful of CTAs keeps hundreds of KiB in flight and the other SMs stay free for the GEMM.
  const bool pull = a.comm_mode == 1;
  if (a.comm_mode == 2) {
    // plain loads and peer stores from every thread of the CTA (no copy engine)
    const uint64_t chunk_bytes = (uint64_t)BM * row_bytes;
    const int split = a.comm_split, ngroups = ncomm / split, grp = cc / split;
    const MtRange r = mt_split(chunk_bytes, split, cc % split, 128);
    if (grp >= ngroups) return;
    for (int w = grp; w < chunks * (n - 1); w += ngroups) {
      {
        const int p = (me + 1 + w / chunks) % n, ci = w % chunks;
        uint8_t* dst = c.heap[p] + a.gather_off + (uint64_t)me * shard_rows * row_bytes;
        uint64_t* cnt = (uint64_t*)(c.heap[p] + a.flags_off) + (uint64_t)me * chunks;
        const uint64_t base = (uint64_t)ci * chunk_bytes + r.lo;
        const uint64_t nvec = (r.hi - r.lo) >> 4;
        for (uint64_t i0 = 0; i0 < nvec; i0 += (uint64_t)kGemmThreads * 8) {
          u128 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint64_t i = i0 + (uint64_t)u * kGemmThreads + threadIdx.x;
            if (i < nvec) v[u] = load128_stream(src + base + (i << 4));
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint64_t i = i0 + (uint64_t)u * kGemmThreads + threadIdx.x;
            if (i < nvec) store128_relaxed_sys(dst + base + (i << 4), v[u]);
          }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
          fence_acq_rel_sys();
          asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(cnt + ci), "l"(1ull) : "memory");
        }
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < COMM_SLOTS; ++s) mbar_init(&cm->full[s], 1);
    cm->abort = 0;
    fence_barrier_init();
    // The comm CTAs form groups of `split` CTAs; a group moves whole 128-row chunks (each CTA a contiguous
    // 1/split of it), the groups work on different chunks at the same time.  Few large contiguous streams
    // per chunk use the link better than every CTA touching every chunk.
    const uint64_t chunk_bytes = (uint64_t)BM * row_bytes;
    const int split = a.comm_split, ngroups = ncomm / split, grp = cc / split;
    const MtRange r = mt_split(chunk_bytes, split, cc % split, 128);
    const uint32_t ppc = (uint32_t)mt_div_up(r.hi - r.lo, COMM_PIECE);   // pieces per chunk for this CTA
    // fan-out push (comm_mode 3): a piece is fetched from local memory once and stored to all n - 1 peers from
    // shared memory, so a CTA reads 1/(n - 1) of what the pairwise push reads and has n - 1 stores in flight per
    // load; the work units are the chunks themselves
    const bool fan = a.comm_mode == 3;
    const uint32_t npairs = fan ? (uint32_t)chunks : (uint32_t)chunks * (uint32_t)(n - 1);   // work units, in push order
    const uint32_t mine = grp < ngroups ? (npairs - grp + ngroups - 1) / ngroups : 0;  // pairs grp, grp+ngroups, ...
    const uint32_t total = ppc * mine;
    volatile int* ab = &cm->abort;
    auto locate = [&](uint32_t i, int& p, int& ci, uint64_t& off, uint32_t& nb) {
      const uint32_t piece = i % ppc, ch_i = grp + (i / ppc) * ngroups;
      ci = (int)(ch_i % chunks);
      p = pull ? mt_mod(me - 1 - (int)(ch_i / chunks), n) : (me + 1 + (int)(ch_i / chunks)) % n;
      off = (uint64_t)ci * chunk_bytes + r.lo + (uint64_t)piece * COMM_PIECE;
      const uint64_t left = r.hi - r.lo - (uint64_t)piece * COMM_PIECE;
      nb = (uint32_t)(left < COMM_PIECE ? left : COMM_PIECE);
    };
    auto signal = [&](uint32_t i) {
      int p, ci;
      uint64_t off;
      uint32_t nb;
      locate(i, p, ci, off, nb);
      if (fan) {
        for (int d = 1; d < n; ++d) {
          uint64_t* pc = (uint64_t*)(c.heap[(me + d) % n] + a.flags_off) + (uint64_t)me * chunks + ci;
          asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(pc), "l"(1ull) : "memory");
        }
        return;
      }
      // push: count on the peer, in my row of its counters; pull: count locally, in the peer's row
      uint64_t* cnt = pull ? (uint64_t*)(c.heap[me] + a.flags_off) + (uint64_t)p * chunks + ci
                           : (uint64_t*)(c.heap[p] + a.flags_off) + (uint64_t)me * chunks + ci;
      // the bulk stores of this chunk have completed (wait_group above); the release orders them before
      // the count.  No proxy fence here: it would drain every copy still in flight.
      asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(cnt), "l"(1ull) : "memory");
    };
    bool ok = ppc > 0;
    for (uint32_t i = 0; ok && i < total + COMM_LAG; ++i) {
      if (i < total) {
        int p, ci;
        uint64_t off;
        uint32_t nb;
        locate(i, p, ci, off, nb);
        const uint32_t s_ = i % COMM_SLOTS;
        // the store that last used this slot (piece i - COMM_SLOTS) must have finished reading it
        if (i >= COMM_SLOTS) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(COMM_SLOTS - COMM_LAG - 1) : "memory");
        mbar_expect_tx(&cm->full[s_], nb);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(smem + (uint64_t)s_ * COMM_PIECE)),
                     "l"(pull ? c.heap[p] + a.shard_off + off : src + off), "r"(nb), "r"(smem_u32(&cm->full[s_]))
                     : "memory");
      }
      if (i >= COMM_LAG) {
        const uint32_t j = i - COMM_LAG;
        int p, ci;
        uint64_t off;
        uint32_t nb;
        locate(j, p, ci, off, nb);
        const uint32_t s_ = j % COMM_SLOTS;
        if (!mbar_wait(&cm->full[s_], (j / COMM_SLOTS) & 1, ab, timeout_ns)) {
          ok = false;
          break;
        }
        if (fan) {
          for (int d = 1; d < n; ++d) {
            uint8_t* pd = c.heap[(me + d) % n] + a.gather_off + (uint64_t)me * shard_rows * row_bytes + off;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(pd),
                         "r"(smem_u32(smem + (uint64_t)s_ * COMM_PIECE)), "r"(nb)
                         : "memory");
          }
        } else {
          uint8_t* dst = pull ? c.heap[me] + a.gather_off + (uint64_t)p * shard_rows * row_bytes + off
                              : c.heap[p] + a.gather_off + (uint64_t)me * shard_rows * row_bytes + off;
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                       "r"(smem_u32(smem + (uint64_t)s_ * COMM_PIECE)), "r"(nb)
                       : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        // A chunk is announced once its last store has COMPLETED (not merely left shared memory).  That
        // takes a round trip to the peer, so announcements trail the stores by COMM_SIGLAG pieces: up to
        // that many stores are in flight per CTA and nothing waits for an acknowledgement it needs now.
        if (j >= COMM_SIGLAG && ((j - COMM_SIGLAG) % ppc) == ppc - 1) {
          asm volatile("cp.async.bulk.wait_group %0;" ::"n"(COMM_SIGLAG) : "memory");
          signal(j - COMM_SIGLAG);
        }
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (ok) {
      for (uint32_t j = total > COMM_SIGLAG ? total - COMM_SIGLAG : 0; j < total; ++j)
        if (j % ppc == ppc - 1) signal(j);
    } else {
      gemm_report(a, lr, MT_WHERE_GEMM_FLAG);
    }
  }
  // pull: the peers read my rows; they must stay untouched until everybody has finished reading
  if (pull) rank_barrier(c, cc, &s_fail);
}

}  // namespace fused
}  // namespace mt
