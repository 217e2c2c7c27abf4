// Persistent bf16 GEMM on the 5th-generation tensor cores, and its two fusions with a collective:
//
//   MODE_PLAIN    C[M,N]  = A[M,K] * B[N,K]^T
//   MODE_AG_GEMM  C[M,N]  = allgather(A_shard)[M,K] * B[N,K]^T       (column-parallel layer, sequence
//                 parallel input): a few "comm" CTAs push this rank's rows into every peer's gathered
//                 buffer chunk by chunk and count each chunk on the peer; the TMA producer of a GEMM CTA
//                 waits for the count of the row block it is about to load.  Rows are consumed in arrival
//                 order (own rows first), so transfer and MMA overlap tile by tile.
//   MODE_GEMM_RS  out[M/n,N] = reduce_scatter(A[M,K_local] * B[N,K_local]^T)   (row-parallel layer):
//                 tiles whose rows belong to other ranks are computed first; the epilogue writes each
//                 partial tile straight into the owner's staging area over NVLink and counts it there;
//                 when a CTA runs out of tiles it turns into a reducer that waits for the partial tiles
//                 of one output tile, sums them in fp32 and writes the result.
//
// One CTA = 192 threads: warp 0 issues TMA loads (4-stage ring of 128x64 A and 256x64 B tiles, 128-byte
// swizzle), warp 1 owns TMEM (512 columns: two 128x256 fp32 accumulators) and issues tcgen05.mma from a
// single thread, warps 2..5 are the epilogue (tcgen05.ld, fp32 -> bf16, transposed through shared
// memory so that global / peer stores are full 128-byte lines).  Every wait is bounded; on expiry the
// CTA records an error, drains, frees its TMEM and returns.
//
// The reference has no counterpart: its README asks that collectives be "fused with other kernels"
// (README.md:5) and stops there.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../device/prims.cuh"
#include "../device/sched.h"
#include "../device/tc_prims.cuh"
#include "fused_schedule.h"
#include "gemm_fused_parts.cuh"
#include "gemm_tc.h"
#include "launch.h"

namespace mt {
using namespace tc;

using namespace fused;

constexpr int BK = 64, UMMA_K = 16, STAGES = 4;
constexpr uint32_t A_TILE_BYTES = BM * BK * 2, B_TILE_BYTES = BN * BK * 2;
constexpr uint32_t STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int EPI_PITCH = 144;                      // bytes per staged row: 64 bf16 + 16 bytes of padding
constexpr uint32_t EPI_BYTES = 4 * 32 * EPI_PITCH;  // 4 epilogue warps x 32 rows
constexpr uint32_t SF_STAGE_BYTES = 1536;  // MXFP8: one 512-byte scale atom for A, two for B, per stage
constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + 256 + STAGES * SF_STAGE_BYTES;
constexpr uint32_t TMEM_COLS = 512;
static_assert(STAGES * STAGE_BYTES >= COMM_SLOTS * COMM_PIECE, "the comm ring reuses the operand stages");

struct SharedCtl {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], drain;
  uint32_t tmem_base;
  int abort;
};

// Tile order: fused_schedule.h (shared with the CTA-pair kernel and the host model).
struct TileCoord {
  int mb, nb, owner;
};
template <int MODE>
__device__ __forceinline__ TileCoord tile_coord(const GemmArgs& a, int lr, int t) {
  static_assert(MODE_PLAIN == MT_TILE_PLAIN && MODE_AG_GEMM == MT_TILE_AG_GEMM && MODE_GEMM_RS == MT_TILE_GEMM_RS, "mode codes");
  const MtTile m = mt_fused_tile(MODE, t, a.M, a.N, a.nranks, a.rank[lr], a.raster, BM, BN);
  TileCoord c;
  c.mb = m.mb;
  c.nb = m.nb;
  c.owner = m.owner;
  return c;
}

template <int MODE, bool FP8>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tc_kernel(const __grid_constant__ GemmMaps maps, GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const int lr = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_TILE_BYTES;
  uint8_t* sEpi = smem + STAGES * STAGE_BYTES;
  SharedCtl* ctl = (SharedCtl*)(sEpi + EPI_BYTES);
  uint8_t* sSF = sEpi + EPI_BYTES + 256;            // MXFP8 scale atoms, SF_STAGE_BYTES per stage
  constexpr int BKE = FP8 ? 128 : 64;                // K elements per stage (128 bytes per row either way)
  constexpr uint32_t ACC = FP8 ? 1 : 2;              // accumulator buffers (MXFP8 needs TMEM columns for scales)
  const int ncomm = MODE == MODE_PLAIN ? 0 : a.ncomm;  // AG: data movers, RS: dedicated reducers
  const int ngemm = gridDim.x - ncomm;
  const uint64_t timeout_ns = a.timeout_ns;

  // ---------------------------------------------------------------- comm CTAs of the all-gather fusion
  if (MODE == MODE_AG_GEMM && (int)blockIdx.x >= ngemm) {
    ag_comm_cta<FP8>(a, lr, blockIdx.x - ngemm, ncomm, smem, (CommCtl*)(sEpi + EPI_BYTES));
    return;
  }

  // ---------------------------------------------------------------- dedicated reducer CTAs
  if (MODE == MODE_GEMM_RS && (int)blockIdx.x >= ngemm) {
    rs_reduce_loop(a, lr);
    return;
  }

  // ---------------------------------------------------------------- GEMM CTAs: set-up
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->acc_full[s], 1);
      mbar_init(&ctl->acc_empty[s], 4);  // one arrival per epilogue warp
    }
    mbar_init(&ctl->drain, 1);
    ctl->abort = 0;
    fence_barrier_init();
    tma_prefetch_desc(&maps.a[lr]);
    tma_prefetch_desc(&maps.b[lr]);
    if (MODE == MODE_AG_GEMM) tma_prefetch_desc(&maps.a2[lr]);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort;

  const int total_tiles = (a.M / BM) * (a.N / BN);
  const int kblocks = a.K / BKE;
  const int first = blockIdx.x;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one lane)
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = first; t < total_tiles && !*abort_flag; t += ngemm) {
        const TileCoord tc_ = tile_coord<MODE>(a, lr, t);
        const CUtensorMap* amap = &maps.a[lr];
        int arow = tc_.mb * BM;
        if (MODE == MODE_AG_GEMM) {
          if (tc_.owner == a.rank[lr]) {
            amap = &maps.a2[lr];  // own rows come straight from the local shard
            arow = tc_.mb * BM - tc_.owner * (a.M / a.nranks);
          } else {
            // rows pushed by `owner`: wait until all comm CTAs of that rank have counted this block in
            const int per = (a.M / a.nranks) / BM;
            const uint64_t* cnt = (const uint64_t*)a.flags_local[lr] + (uint64_t)tc_.owner * per + (tc_.mb % per);
            const uint64_t want = a.epoch * (uint64_t)a.comm_split;  // every CTA of the group counts the chunk once
            uint32_t spins = 0;
            uint64_t t0 = 0;
            while (load64_acquire_sys(cnt) < want) {
              if ((++spins & 0xffu) == 0) {
                const uint64_t now = globaltimer();
                if (t0 == 0) t0 = now;
                else if (now - t0 > timeout_ns || *abort_flag) {
                  *abort_flag = 1;
                  gemm_report(a, lr, MT_WHERE_GEMM_FLAG);
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
          if (!mbar_wait(&ctl->empty[s], ph ^ 1, abort_flag, timeout_ns)) break;
          mbar_expect_tx(&ctl->full[s], STAGE_BYTES + (FP8 ? SF_STAGE_BYTES : 0));
          tma_load_2d(sA + s * A_TILE_BYTES, amap, kb * BKE, arow, &ctl->full[s]);
          tma_load_2d(sB + s * B_TILE_BYTES, &maps.b[lr], kb * BKE, tc_.nb * BN, &ctl->full[s]);
          if (FP8) {
            const uint8_t* fa = (const uint8_t*)a.sfa[lr] + ((uint64_t)tc_.mb * kblocks + kb) * 512;
            const uint8_t* fb = (const uint8_t*)a.sfb[lr] + ((uint64_t)(tc_.nb * 2) * kblocks + kb) * 512;
            uint8_t* sf = sSF + s * SF_STAGE_BYTES;
            bulk_load_1d(sf, fa, 512, &ctl->full[s]);
            bulk_load_1d(sf + 512, fb, 512, &ctl->full[s]);
            bulk_load_1d(sf + 1024, fb + (uint64_t)kblocks * 512, 512, &ctl->full[s]);
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
    // ------------------------------------------------------------ MMA issuer (one lane)
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      uint32_t it = 0, tile_i = 0;
      for (int t = first; t < total_tiles && !*abort_flag; t += ngemm, ++tile_i) {
        const uint32_t as = tile_i % ACC, aph = (tile_i / ACC) & 1;
        if (!mbar_wait(&ctl->acc_empty[as], aph ^ 1, abort_flag, timeout_ns)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(&ctl->full[s], ph, abort_flag, timeout_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = make_smem_desc_sw128(sA + s * A_TILE_BYTES);
          const uint64_t db = make_smem_desc_sw128(sB + s * B_TILE_BYTES);
          if (FP8) {
            // scales of this stage -> TMEM (the tensor pipe runs copies and MMAs in issue order, so the
            // same columns serve every stage), then one MMA per 32-element K block with its scale byte
            const uint32_t tsfa = tmem_base + 256, tsfb = tmem_base + 260;
            const uint8_t* sf = sSF + s * SF_STAGE_BYTES;
            tmem_cp_sf(tsfa, make_smem_desc_sf(sf));
            tmem_cp_sf(tsfb, make_smem_desc_sf(sf + 512));
            tmem_cp_sf(tsfb + 4, make_smem_desc_sf(sf + 1024));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_mxfp8(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), make_idesc_mxfp8(BM, BN, k, k), tsfa, tsfb,
                         (kb > 0 || k > 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&ctl->empty[s]);  // the stage is free once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&ctl->acc_full[as]);
      }
      // no MMA may still be writing TMEM when it is freed, on the normal path or after an abort
      umma_commit(&ctl->drain);
      mbar_wait(&ctl->drain, 0, abort_flag, timeout_ns);
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint8_t* stg = sEpi + (warp - 2) * 32 * EPI_PITCH;
    uint32_t tile_i = 0;
    for (int t = first; t < total_tiles; t += ngemm, ++tile_i) {
      const uint32_t as = tile_i % ACC, aph = (tile_i / ACC) & 1;
      if (!mbar_wait(&ctl->acc_full[as], aph, abort_flag, timeout_ns)) break;
      tc_fence_after();
      const TileCoord tc_ = tile_coord<MODE>(a, lr, t);
      // destination of this tile's rows
      uint8_t* dst;
      uint64_t ld_bytes;
      if (MODE == MODE_GEMM_RS) {
        // partial tile -> staging[my rank] of the owner (peer memory unless the owner is this rank)
        // The staging area is tile-major: [source rank][row block][column block][128 x 256], so a CTA
        // writes one contiguous 64 KiB region (contiguous streams use the link far better than rows
        // interleaved with other CTAs' rows).
        const MtDevComm& c = a.comms[lr];
        const int per = (a.M / a.nranks) / BM;
        ld_bytes = (uint64_t)BN * 2;
        dst = c.heap[tc_.owner] + a.stage_off +
              (((uint64_t)a.rank[lr] * per + (tc_.mb % per)) * (a.N / BN) + tc_.nb) * (uint64_t)(BM * BN * 2);
      } else {
        ld_bytes = (uint64_t)a.ldc * 2;
        dst = (uint8_t*)a.c[lr] + (uint64_t)tc_.mb * BM * ld_bytes + (uint64_t)tc_.nb * BN * 2;
      }
      dst += (uint64_t)(q * 32) * ld_bytes;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN;
      // 4 rows per pass of 8 lanes x 16 bytes: full 128-byte lines on the wire
      auto store_block = [&](int cb) {
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          const int rr = p * 4 + (lane >> 3), c16 = lane & 7;
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
        // One accumulator only (the scales take TMEM columns), so the MMA warp waits for this drain: pull
        // the whole row into registers as packed bf16 first, hand the accumulator back, and only then go
        // through shared memory to global memory, which overlaps the next tile's MMAs.
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
        if (lane == 0) mbar_arrive(&ctl->acc_empty[as]);
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
        for (int cb = 0; cb < BN / 64; ++cb) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + cb * 64, r0);
          tmem_ld_32x32(taddr + cb * 64 + 32, r1);
          tmem_ld_wait();
          // fp32 -> bf16, row `lane` of the staging tile (conflict-free: pitch 144 bytes)
          uint4* row = (uint4*)(stg + lane * EPI_PITCH);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
            o.x = *(uint32_t*)&p0; o.y = *(uint32_t*)&p1; o.z = *(uint32_t*)&p2; o.w = *(uint32_t*)&p3;
            row[j] = o;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
            o.x = *(uint32_t*)&p0; o.y = *(uint32_t*)&p1; o.z = *(uint32_t*)&p2; o.w = *(uint32_t*)&p3;
            row[4 + j] = o;
          }
          __syncwarp();
          store_block(cb);
          __syncwarp();
        }
        // accumulator drained: hand it back to the MMA warp
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc_empty[as]);
      }
      if (MODE == MODE_GEMM_RS) {
        // count this warp's quarter of the tile on the owner (release: the stores above come first)
        if (lane == 0) {
          const MtDevComm& c = a.comms[lr];
          const int per = (a.M / a.nranks) / BM;
          uint64_t* cnt = (uint64_t*)(c.heap[tc_.owner] + a.flags_off) +
                          ((uint64_t)a.rank[lr] * per + (tc_.mb % per)) * (a.N / BN) + tc_.nb;
          asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(cnt), "l"(1ull) : "memory");
        }
      }
    }
  }

  // ---------------------------------------------------------------- tear-down
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) {
    gemm_report(a, lr, MT_WHERE_GEMM_FLAG);
  }

  // ---------------------------------------------------------------- reducer phase of GEMM -> reduce-scatter
  if (MODE == MODE_GEMM_RS) {
    if (*abort_flag) return;
    rs_reduce_loop(a, lr);
  }
}

template <int MODE, bool FP8>
static cudaError_t launch_mode(const GemmMaps& maps, const GemmArgs& a, int nctas, int nlocal, cudaStream_t s) {
  static bool attr_set = false;
  const void* fn = (const void*)gemm_tc_kernel<MODE, FP8>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  GemmMaps m = maps;
  GemmArgs args = a;
  void* p[] = {(void*)&m, (void*)&args};
  count_launch();
  if (nlocal > 1) return cudaLaunchCooperativeKernel(fn, dim3(nctas, nlocal), dim3(kGemmThreads), p, SMEM_BYTES, s);
  return cudaLaunchKernel(fn, dim3(nctas, nlocal), dim3(kGemmThreads), p, SMEM_BYTES, s);
}

cudaError_t launch_gemm_tc(int mode, const GemmMaps& maps, const GemmArgs& a, int nctas, int nlocal, cudaStream_t s,
                           bool fp8) {
  if (fp8) {
    switch (mode) {
      case MODE_PLAIN: return launch_mode<MODE_PLAIN, true>(maps, a, nctas, nlocal, s);
      case MODE_AG_GEMM: return launch_mode<MODE_AG_GEMM, true>(maps, a, nctas, nlocal, s);
      case MODE_GEMM_RS: return launch_mode<MODE_GEMM_RS, true>(maps, a, nctas, nlocal, s);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (mode) {
    case MODE_PLAIN: return launch_mode<MODE_PLAIN, false>(maps, a, nctas, nlocal, s);
    case MODE_AG_GEMM: return launch_mode<MODE_AG_GEMM, false>(maps, a, nctas, nlocal, s);
    case MODE_GEMM_RS: return launch_mode<MODE_GEMM_RS, false>(maps, a, nctas, nlocal, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace mt
