// GEMM on CTA pairs: C[M, N] = A[M, K] * B[N, K]^T with tcgen05.mma.cta_group::2.
//
// Two CTAs of one cluster (neighbouring SMs) compute one 256 x 256 tile.  Each CTA stages 128 rows of A and
// 128 rows of B per K block, so the tensor cores of both SMs read every B row from ONE shared memory only:
// per SM and MMA, the shared-memory traffic (TMA writes + operand reads) drops from 24 KiB to 16 KiB compared
// with the single-CTA 128 x 256 tile of gemm_tc.cu, and a stage takes 32 KiB instead of 48, which pays for a
// 6-deep ring.  The leader CTA (cluster rank 0) issues every MMA; the accumulator rows [0, 128) live in the
// leader's TMEM and [128, 256) in the peer's, and each CTA's epilogue warps drain their own half.
//
//   warp 0 (both CTAs)  TMA producer: own halves of A and B (and the MXFP8 scale atoms) into own shared
//                       memory; the bytes of both CTAs are counted on the LEADER's "stage full" barrier
//   warp 1 (leader)     one lane issues tcgen05.mma for the pair and commits to the leader's "stage empty" and
//                       "accumulator full" barriers; the leader's producer / first epilogue warp pass each
//                       of these on to the peer's barrier with a remote mbarrier arrive
//   warps 2..5 (both)   epilogue: TMEM -> registers -> bf16 -> shared memory -> global memory; every warp
//                       arrives on the leader's "accumulator empty" barrier (8 arrivals per tile)
//
// Every wait is bounded; on expiry the CTA raises its abort flag, all roles leave their loops, both CTAs meet
// at the closing cluster barrier (so neither exits while the other may still signal into it), TMEM is
// released and a device-side error word is set for the host.  No load is replicated across the cluster.
//
// Modes (as in gemm_tc.cu): the plain GEMM; all-gather -> GEMM, where extra CTAs of the grid move the peers' rows
// into local memory and each producer waits for the arrival counter of its own 128 rows; GEMM -> reduce-scatter,
// where the epilogue stores partial tiles into the row owner's staging area over NVLink and extra CTAs (then
// all CTAs) reduce this rank's rows.  The comm and reducer CTAs are the ones of gemm_tc.cu
// (gemm_fused_parts.cuh); they come in whole clusters and never take part in a cluster barrier.
//
// The reference has no compute kernels (README.md:5 only asks that collectives fuse with others).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../device/prims.cuh"
#include "../device/tc_prims.cuh"
#include "fused_schedule.h"
#include "gemm_fused_parts.cuh"
#include "gemm_tc.h"
#include "launch.h"

namespace mt {
using namespace tc;
namespace pair {

constexpr int BMC = 128;   // A rows (and accumulator rows) per CTA
constexpr int BM2 = 256;   // rows of the pair's tile
constexpr int BN = 256;    // columns of the tile
constexpr int BNC = 128;   // B rows staged by each CTA
constexpr int STAGES = 6;
constexpr int kThreads = 192;
constexpr uint32_t A_BYTES = BMC * 128, B_BYTES = BNC * 128;  // rows of 128 bytes (64 bf16 or 128 fp8)
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_PITCH = 144;
constexpr uint32_t EPI_BYTES = 4 * 32 * EPI_PITCH;
constexpr uint32_t SF_STAGE_BYTES = 1536;  // MXFP8: scale atom of the CTA's A rows + two atoms for all 256 B rows
constexpr uint32_t CTL_BYTES = 512;
constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + CTL_BYTES + STAGES * SF_STAGE_BYTES;
constexpr uint32_t TMEM_COLS = 512;
static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA");

struct Ctl {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], drain;
  uint32_t tmem_base;
  int abort;
};
static_assert(sizeof(Ctl) <= CTL_BYTES && sizeof(fused::CommCtl) <= CTL_BYTES, "control block");
static_assert(STAGES * STAGE_BYTES >= fused::COMM_SLOTS * fused::COMM_PIECE, "the comm ring reuses the operand stages");
static_assert(kThreads == fused::kGemmThreads, "comm and reducer code assumes this block size");

__device__ int g_pair_error;  // set when a wait of this kernel expired (read by mt_gemm_pair_error)

__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint64_t timeout_ns) {
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

// Tile order: fused_schedule.h with 256-row tiles (mb, jb count 256-row blocks).
using Tile = MtTile;
template <int MODE, int TILE_N>
__device__ __forceinline__ Tile tile_of(const GemmArgs& a, int lr, int t) {
  static_assert(MODE_PLAIN == MT_TILE_PLAIN && MODE_AG_GEMM == MT_TILE_AG_GEMM && MODE_GEMM_RS == MT_TILE_GEMM_RS, "mode codes");
  return mt_fused_tile(MODE, t, a.M, a.N, a.nranks, a.rank[lr], a.raster, BM2, TILE_N);
}

// TILE_N: columns of a tile, 256 or 224.  224 exists for the wave count: 8192 x 1792 (the Llama-3-8B up projection on
// 8 ranks) is 224 tiles of 256 x 256, 3.03 waves on 74 clusters, i.e. a fourth wave for two tiles; as 256 tiles of
// 256 x 224 it is four waves of tiles that are an eighth smaller.  bf16 only (the MXFP8 scale atoms cover 128
// rows of B) and not for GEMM -> reduce-scatter (its staging layout is in 256-column tiles).
template <int MODE, bool FP8, int TILE_N>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ PairSfMaps sfmaps, GemmArgs a) {
  static_assert(TILE_N == 256 || (TILE_N == 224 && !FP8 && MODE != MODE_GEMM_RS), "tile widths");
  constexpr int BN = TILE_N, BNC = TILE_N / 2;             // shadow the 256-column constants of the namespace
  constexpr uint32_t B_BYTES = BNC * 128;                   // a multiple of 1024: whole 128-byte swizzle atoms
  extern __shared__ uint8_t smem_raw[];
  const int lr = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the same offsets in both CTAs: the MMA descriptors name shared memory of the pair by offset
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* sEpi = smem + STAGES * STAGE_BYTES;
  Ctl* ctl = (Ctl*)(sEpi + EPI_BYTES);
  uint8_t* sSF = sEpi + EPI_BYTES + CTL_BYTES;
  constexpr int BKE = FP8 ? 128 : 64;    // K elements per stage
  constexpr uint32_t ACC = FP8 ? 1 : 2;  // accumulator buffers (MXFP8 keeps TMEM columns for the scales)
  const uint32_t cr = cluster_ctarank();
  const bool leader = cr == 0;
  const int nextra = MODE == MODE_PLAIN ? 0 : a.ncomm;  // AG: data movers, RS: dedicated reducers (whole clusters)
  const int ngemm = (int)gridDim.x - nextra;
  const int cluster_id = blockIdx.x >> 1, nclusters = ngemm >> 1;
  const uint64_t timeout_ns = a.timeout_ns;

  if (MODE == MODE_AG_GEMM && (int)blockIdx.x >= ngemm) {
    fused::ag_comm_cta<FP8>(a, lr, (int)blockIdx.x - ngemm, nextra, smem, (fused::CommCtl*)(sEpi + EPI_BYTES));
    return;
  }
  if (MODE == MODE_GEMM_RS && (int)blockIdx.x >= ngemm) {
    fused::rs_reduce_loop(a, lr);
    return;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);   // the leader's producer arrives once with the byte count of both CTAs
      mbar_init(&ctl->empty[s], 1);  // leader: commit of the MMA thread; peer: arrive forwarded by the leader
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->acc_full[s], 1);
      mbar_init(&ctl->acc_empty[s], 8);  // 4 epilogue warps of each CTA
    }
    mbar_init(&ctl->drain, 1);
    ctl->abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&maps.a[lr]);
    tma_prefetch_desc(&maps.b[lr]);
  }
  if (warp == 1) {
    tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anybody signals across
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort;

  const int tiles = (a.M / BM2) * (a.N / BN);
  const int kblocks = a.K / BKE;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one lane, both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = cluster_id; t < tiles && !*abort_flag; t += nclusters) {
        const Tile tc_ = tile_of<MODE, BN>(a, lr, t);
        int arow = tc_.mb * BM2 + (int)cr * BMC;
        const int brow = tc_.nb * BN + (int)cr * BNC;
        const int sfa_row = tc_.mb * 2 + (int)cr;  // 128-row block of A in the (gathered) scale tensor
        const CUtensorMap* amap = &maps.a[lr];
        if (MODE == MODE_AG_GEMM) {
          if (tc_.owner == a.rank[lr]) {
            amap = &maps.a2[lr];  // own rows come straight from the local shard
            arow -= tc_.owner * (a.M / a.nranks);
          } else {
            // this CTA's 128 rows were pushed by `owner`: wait until its comm CTAs have counted the block in
            const int per = (a.M / a.nranks) / BMC;
            const uint64_t* cnt = (const uint64_t*)a.flags_local[lr] + (uint64_t)tc_.owner * per + (tc_.jb * 2 + (int)cr);
            const uint64_t want = a.epoch * (uint64_t)a.comm_split;
            uint32_t spins = 0;
            uint64_t t0 = 0;
            while (load64_acquire_sys(cnt) < want) {
              if ((++spins & 0xffu) == 0) {
                const uint64_t now = globaltimer();
                if (t0 == 0) t0 = now;
                else if (now - t0 > timeout_ns || *abort_flag) {
                  *abort_flag = 1;
                  fused::gemm_report(a, lr, MT_WHERE_GEMM_FLAG);
                  break;
                }
              }
            }
            if (*abort_flag) break;
            fence_proxy_async_global();  // peer stores (generic proxy) before our TMA reads (async proxy)
          }
        }
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!wait_bar(&ctl->empty[s], ph ^ 1, abort_flag, timeout_ns)) break;
          // the MMA thread's commit lands on the leader's barrier only: pass it on to the peer's producer
          if (leader && it >= (uint32_t)STAGES) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->empty[s]), 1));
          const uint32_t full0 = map_to_cta(smem_u32(&ctl->full[s]), 0);
          if (leader) mbar_expect_tx(&ctl->full[s], 2 * (A_BYTES + B_BYTES + (FP8 ? SF_STAGE_BYTES : 0)));
          tma_load_2d_pair(sA + s * A_BYTES, amap, kb * BKE, arow, full0);
          tma_load_2d_pair(sB + s * B_BYTES, &maps.b[lr], kb * BKE, brow, full0);
          if (FP8) {
            // scale atoms are rows of a [atoms, 128 x u32] tensor: atom (row block of 128, K block of 128)
            uint8_t* sf = sSF + s * SF_STAGE_BYTES;
            tma_load_2d_pair(sf, &sfmaps.sfa[lr], 0, sfa_row * kblocks + kb, full0);
            tma_load_2d_pair(sf + 512, &sfmaps.sfb[lr], 0, (tc_.nb * 2) * kblocks + kb, full0);
            tma_load_2d_pair(sf + 1024, &sfmaps.sfb[lr], 0, (tc_.nb * 2 + 1) * kblocks + kb, full0);
          }
        }
      }
      if (*abort_flag) {
        // copies this thread issued may still be landing in shared memory: give them a bounded time
        const uint64_t t0 = globaltimer();
        while (globaltimer() - t0 < 100000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (one lane of the leader)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM2, BN);
      uint32_t it = 0, tile_i = 0;
      for (int t = cluster_id; t < tiles && !*abort_flag; t += nclusters, ++tile_i) {
        const uint32_t as = tile_i % ACC, aph = (tile_i / ACC) & 1;
        if (!wait_bar(&ctl->acc_empty[as], aph ^ 1, abort_flag, timeout_ns)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!wait_bar(&ctl->full[s], ph, abort_flag, timeout_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = make_smem_desc_sw128(sA + s * A_BYTES);
          const uint64_t db = make_smem_desc_sw128(sB + s * B_BYTES);
          if (FP8) {
            const uint32_t tsfa = tmem_base + 256, tsfb = tmem_base + 260;
            const uint8_t* sf = sSF + s * SF_STAGE_BYTES;
            tmem_cp_sf_pair(tsfa, make_smem_desc_sf(sf));
            tmem_cp_sf_pair(tsfb, make_smem_desc_sf(sf + 512));
            tmem_cp_sf_pair(tsfb + 4, make_smem_desc_sf(sf + 1024));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_mxfp8_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), make_idesc_mxfp8(BM2, BN, k, k), tsfa,
                              tsfb, (kb > 0 || k > 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // the stage is free (in both CTAs) once these MMAs have read it
          umma_commit_pair(smem_u32(&ctl->empty[s]));
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(&ctl->acc_full[as]));
      }
      // no MMA may still be running when TMEM is freed, on the normal path or after an abort
      umma_commit_pair(smem_u32(&ctl->drain));
      wait_bar(&ctl->drain, 0, abort_flag, timeout_ns);
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5, both CTAs)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint8_t* stg = sEpi + (warp - 2) * 32 * EPI_PITCH;
    uint32_t tile_i = 0;
    for (int t = cluster_id; t < tiles; t += nclusters, ++tile_i) {
      const uint32_t as = tile_i % ACC, aph = (tile_i / ACC) & 1;
      if (!wait_bar(&ctl->acc_full[as], aph, abort_flag, timeout_ns)) break;
      // the commit lands on the leader's barrier only: its first epilogue warp passes it on to the peer
      if (leader && warp == 2 && lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->acc_full[as]), 1));
      tc_fence_after();
      const Tile tc_ = tile_of<MODE, BN>(a, lr, t);
      // destination of this CTA's 128 rows of the tile
      uint8_t* dst;
      uint64_t ld_bytes;
      uint64_t* rs_cnt = nullptr;
      if (MODE == MODE_GEMM_RS) {
        // partial tile -> staging[my rank] of the owner (peer memory unless the owner is this rank), tile-major:
        // [source rank][128-row block][column block][128 x 256], one contiguous 64 KiB region per CTA and tile
        const MtDevComm& c = a.comms[lr];
        const int per = (a.M / a.nranks) / BMC;
        const uint64_t slot = ((uint64_t)a.rank[lr] * per + (tc_.jb * 2 + (int)cr)) * (a.N / BN) + tc_.nb;
        ld_bytes = (uint64_t)BN * 2;
        dst = c.heap[tc_.owner] + a.stage_off + slot * (uint64_t)(BMC * BN * 2);
        rs_cnt = (uint64_t*)(c.heap[tc_.owner] + a.flags_off) + slot;
      } else {
        ld_bytes = (uint64_t)a.ldc * 2;
        dst = (uint8_t*)a.c[lr] + (uint64_t)(tc_.mb * BM2 + (int)cr * BMC) * ld_bytes + (uint64_t)tc_.nb * BN * 2;
      }
      dst += (uint64_t)(q * 32) * ld_bytes;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN;
      const uint32_t acc_empty0 = map_to_cta(smem_u32(&ctl->acc_empty[as]), 0);
      // 4 rows per pass of 8 lanes x 16 bytes: full 128-byte lines
      // `nchunk` 16-byte pieces per row: 8 for a full block of 64 columns, 4 for the last half block of a 224 tile
      auto store_block = [&](int cb, int nchunk = 8) {
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          const int rr = p * 4 + (lane >> 3), c16 = lane & 7;
          if (c16 >= nchunk) continue;
          const uint4 v = *(const uint4*)(stg + rr * EPI_PITCH + c16 * 16);
          uint8_t* g = dst + (uint64_t)rr * ld_bytes + cb * 128 + c16 * 16;
          if (MODE == MODE_GEMM_RS) {
            u128 w;
            w.x = (uint64_t)v.x | ((uint64_t)v.y << 32);
            w.y = (uint64_t)v.z | ((uint64_t)v.w << 32);
            store128_relaxed_sys(g, w);
          } else {
            *(uint4*)g = v;
          }
        }
      };
      if constexpr (FP8) {
        // single accumulator: drain it into registers (packed bf16) first and hand it back, then store
        uint32_t pk[BN / 2];
#pragma unroll
        for (int cb = 0; cb < BN / 64; ++cb) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + cb * 64, r0);
          tmem_ld_32x32(taddr + cb * 64 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r0[2 * j]), __uint_as_float(r0[2 * j + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1]));
            pk[cb * 32 + j] = *(uint32_t*)&p0;
            pk[cb * 32 + 16 + j] = *(uint32_t*)&p1;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty0);
#pragma unroll
        for (int cb = 0; cb < BN / 64; ++cb) {
          uint4* row = (uint4*)(stg + lane * EPI_PITCH);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            row[j] = make_uint4(pk[cb * 32 + 4 * j], pk[cb * 32 + 4 * j + 1], pk[cb * 32 + 4 * j + 2], pk[cb * 32 + 4 * j + 3]);
          __syncwarp();
          store_block(cb);
          __syncwarp();
        }
      } else {
#pragma unroll 1
        for (int cb = 0; cb < (BN + 63) / 64; ++cb) {
          uint32_t r0[32], r1[32];
          const bool half = cb * 64 + 32 >= BN;   // only 32 columns left (224 = 3 x 64 + 32)
          tmem_ld_32x32(taddr + cb * 64, r0);
          if (!half) tmem_ld_32x32(taddr + cb * 64 + 32, r1);
          tmem_ld_wait();
          uint4* row = (uint4*)(stg + lane * EPI_PITCH);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
            row[j] = make_uint4(*(uint32_t*)&p0, *(uint32_t*)&p1, *(uint32_t*)&p2, *(uint32_t*)&p3);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
            row[4 + j] = make_uint4(*(uint32_t*)&p0, *(uint32_t*)&p1, *(uint32_t*)&p2, *(uint32_t*)&p3);
          }
          __syncwarp();
          store_block(cb, half ? 4 : 8);
          __syncwarp();
        }
        // accumulator drained: hand it back to the leader's MMA thread
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty0);
      }
      if (MODE == MODE_GEMM_RS) {
        // count this warp's quarter of the partial tile on the owner (release: the stores above come first)
        __syncwarp();
        if (lane == 0) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(rs_cnt), "l"(1ull) : "memory");
      }
    }
  }

  // ---------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) {
    // tell the peer (it would notice by itself after its own time limit) and the host
    st_cluster_u32(map_to_cta(smem_u32(&ctl->abort), cr ^ 1), 1u);
    atomicExch(&g_pair_error, 1);
    if (MODE != MODE_PLAIN) fused::gemm_report(a, lr, MT_WHERE_GEMM_FLAG);
  }
  cluster_sync_all();  // neither CTA leaves, or frees TMEM, while the other may still signal into it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  // ---------------------------------------------------------------- reducer phase of GEMM -> reduce-scatter
  if (MODE == MODE_GEMM_RS) {
    if (*abort_flag) return;
    fused::rs_reduce_loop(a, lr);
  }
}

}  // namespace pair

static const void* pair_fn(int mode, bool fp8, int bn = 256) {
  if (bn == 224) {
    if (fp8) return nullptr;
    if (mode == MODE_PLAIN) return (const void*)pair::gemm_pair_kernel<MODE_PLAIN, false, 224>;
    if (mode == MODE_AG_GEMM) return (const void*)pair::gemm_pair_kernel<MODE_AG_GEMM, false, 224>;
    return nullptr;
  }
  switch (mode * 2 + (fp8 ? 1 : 0)) {
    case MODE_PLAIN * 2: return (const void*)pair::gemm_pair_kernel<MODE_PLAIN, false, 256>;
    case MODE_PLAIN * 2 + 1: return (const void*)pair::gemm_pair_kernel<MODE_PLAIN, true, 256>;
    case MODE_AG_GEMM * 2: return (const void*)pair::gemm_pair_kernel<MODE_AG_GEMM, false, 256>;
    case MODE_AG_GEMM * 2 + 1: return (const void*)pair::gemm_pair_kernel<MODE_AG_GEMM, true, 256>;
    case MODE_GEMM_RS * 2: return (const void*)pair::gemm_pair_kernel<MODE_GEMM_RS, false, 256>;
    case MODE_GEMM_RS * 2 + 1: return (const void*)pair::gemm_pair_kernel<MODE_GEMM_RS, true, 256>;
    default: return nullptr;
  }
}

// Clusters of this kernel that the device can hold at once.  The kernel is persistent (cluster i takes tiles
// i, i + n, ...), so a grid with more clusters than fit would run its tail after the rest has finished.
int gemm_pair_max_clusters(int mode, bool fp8, int bn) {
  static int cached[12] = {};
  const void* fn = pair_fn(mode, fp8, bn);
  if (!fn) return 0;
  int& slot = cached[(mode * 2 + (fp8 ? 1 : 0)) * 2 + (bn == 224 ? 1 : 0)];
  if (slot > 0) return slot;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES) != cudaSuccess) return 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(sms & ~1);
  cfg.blockDim = dim3(pair::kThreads);
  cfg.dynamicSmemBytes = pair::SMEM_BYTES;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = 2;
  at.val.clusterDim.y = 1;
  at.val.clusterDim.z = 1;
  cfg.attrs = &at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = sms / 2;
  }
  if (const char* e = getenv("MINTCCL_DEBUG")) {
    if (strcmp(e, "info") == 0 || strcmp(e, "trace") == 0 || atoi(e) > 0)  // same levels as the Python side
      fprintf(stderr, "[mintccl] pair GEMM (mode %d, %s): %d clusters of 2 CTAs fit on %d SMs\n", mode, fp8 ? "mxfp8" : "bf16", n, sms);
  }
  slot = n;
  return n;
}

// Grid: 2 * nclusters GEMM CTAs followed by a.ncomm comm / reducer CTAs (even), times nlocal emulated ranks.
cudaError_t launch_gemm_pair(int mode, const GemmMaps& maps, const PairSfMaps& sf, const GemmArgs& a, int nclusters,
                             int nlocal, cudaStream_t s, bool fp8, int bn) {
  const void* fn = pair_fn(mode, fp8, bn);
  if (!fn) return cudaErrorInvalidValue;
  const int fit = gemm_pair_max_clusters(mode, fp8, bn);  // also sets the shared-memory attribute once
  if (fit <= 0) return cudaErrorInvalidValue;
  const int extra = mode == MODE_PLAIN ? 0 : a.ncomm;
  if (extra & 1) return cudaErrorInvalidValue;
  if ((nclusters + extra / 2) * nlocal > fit) nclusters = fit / nlocal - extra / 2;
  if (nclusters < 1) return cudaErrorInvalidValue;
  GemmMaps m = maps;
  PairSfMaps sm = sf;
  GemmArgs args = a;
  void* p[] = {(void*)&m, (void*)&sm, (void*)&args};
  count_launch();
  const dim3 grid(2 * nclusters + extra, nlocal);
  if (nlocal == 1) return cudaLaunchKernel(fn, grid, dim3(pair::kThreads), p, pair::SMEM_BYTES, s);
  // emulated ranks wait on each other inside one grid: every CTA has to be resident
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = dim3(pair::kThreads);
  cfg.dynamicSmemBytes = pair::SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeCooperative;
  at.val.cooperative = 1;
  cfg.attrs = &at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelExC(&cfg, fn, p);
}

int gemm_pair_error() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, pair::g_pair_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace mt
