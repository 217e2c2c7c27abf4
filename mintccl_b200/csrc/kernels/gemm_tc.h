// Arguments of the tcgen05 GEMM kernels (plain, all-gather -> GEMM, GEMM -> reduce-scatter).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "../device/layout.h"

namespace mt {

enum GemmMode : int { MODE_PLAIN = 0, MODE_AG_GEMM = 1, MODE_GEMM_RS = 2 };

// TMA descriptors, one set per local rank (index 0 outside single-GPU emulation).
struct GemmMaps {
  CUtensorMap a[MT_MAX_RANKS];   // A operand: [M, K] (AG_GEMM: the gathered buffer)
  CUtensorMap b[MT_MAX_RANKS];   // B operand: [N, K]
  CUtensorMap a2[MT_MAX_RANKS];  // AG_GEMM: this rank's own rows [M / n, K]
};

struct GemmArgs {
  void* c[MT_MAX_RANKS];               // output: C [M, ldc] (GEMM_RS: this rank's rows [M / n, N])
  const void* a_local[MT_MAX_RANKS];   // AG_GEMM: own rows, pushed to the peers by the comm CTAs
  const void* flags_local[MT_MAX_RANKS];  // AG_GEMM: this rank's arrival counters (local view)
  void* status[MT_MAX_RANKS];          // MtStatus of the rank (or null)
  const void* sfa[MT_MAX_RANKS];       // MXFP8: scales of A, tiled [M / 128][K / 128][512 bytes]
  const void* sfb[MT_MAX_RANKS];       // MXFP8: scales of B, tiled [N / 128][K / 128][512 bytes]
  const MtDevComm* comms;              // device descriptors (fused modes)
  int32_t rank[MT_MAX_RANKS];
  int32_t M, N, K, ldc;
  int32_t nranks;
  int32_t ncomm;                       // AG_GEMM: CTAs that move data instead of computing; GEMM_RS: reducers
  int32_t comm_mode;                   // AG_GEMM: 0 copy-engine push (one peer per piece), 1 copy-engine pull, 2 push with plain stores,
                                       // 3 copy-engine fan-out push (every piece to all peers)
  int32_t comm_split;                  // AG_GEMM: comm CTAs that share one 128-row chunk
  int32_t raster;                      // plain GEMM: row blocks per group of the tile order (<= 1: row-major)
  uint64_t shard_off;                  // AG_GEMM pull: heap offset of every rank's own rows
  uint64_t gather_off;                 // AG_GEMM: heap offset of the gathered A buffer [M, K]
  uint64_t flags_off;                  // heap offset of the arrival counters
  uint64_t stage_off;                  // GEMM_RS: heap offset of the partial tiles [n, M / n, N]
  uint64_t epoch;                      // call number on these counters (they only ever grow)
  uint64_t timeout_ns;
};

cudaError_t launch_gemm_tc(int mode, const GemmMaps& maps, const GemmArgs& a, int nctas, int nlocal, cudaStream_t s,
                           bool fp8 = false);

// ---- GEMM on CTA pairs (gemm_tc2.cu): one 256 x 256 tile per cluster of two CTAs, same modes and arguments ----
// GemmMaps for this kernel: boxes of 128 rows x 128 bytes for A and for B (each CTA of a pair loads half of B).
struct PairSfMaps {
  CUtensorMap sfa[MT_MAX_RANKS];  // MXFP8: tiled scales of (the gathered) A as [atoms, 128] u32, box = one 512-byte atom
  CUtensorMap sfb[MT_MAX_RANKS];  // same for B
};
// bn: columns of a tile, 256, or 224 (bf16, plain GEMM and all-gather -> GEMM only; the map of B then has boxes of
// 112 rows)
cudaError_t launch_gemm_pair(int mode, const GemmMaps& maps, const PairSfMaps& sf, const GemmArgs& a, int nclusters,
                             int nlocal, cudaStream_t s, bool fp8, int bn = 256);
int gemm_pair_max_clusters(int mode, bool fp8, int bn = 256);
int gemm_pair_error();   // 1 after a wait of the pair kernel expired (synchronises), -1 on a CUDA error

}  // namespace mt
