// Host side of the tcgen05 GEMM kernels: TMA descriptors, argument checks, launches.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include <string>

#include "../kernels/gemm_tc.h"
#include "../kernels/mxfp8.h"
#include "comm_internal.h"

using mthost::fail;

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kPairDefault = 1;  // plain GEMMs on CTA pairs unless MINTCCL_GEMM_PAIR says otherwise

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, K] bf16 row-major, tiles of box_rows x 64 elements, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows, bool fp8 = false) {
  static EncodeTiledFn enc = (EncodeTiledFn)mthost::driver_entry("cuTensorMapEncodeTiled");
  if (!enc) return fail("cuTensorMapEncodeTiled not available");
  const uint64_t esz = fp8 ? 1 : 2;
  if (((uintptr_t)base & 15) || (K * esz) % 16) return fail("GEMM operands must be 16-byte aligned with rows a multiple of 16 bytes");
  cuuint64_t dims[2] = {K, rows};
  cuuint64_t strides[1] = {K * esz};
  cuuint32_t box[2] = {(cuuint32_t)(fp8 ? 128 : kBK), box_rows};  // 128 bytes per row either way
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed: CUresult " + std::to_string((int)r));
  return 0;
}

// Tiled MXFP8 scales as a [atoms, 128] tensor of 32-bit words: one box = one 512-byte atom.
int make_sf_map(CUtensorMap* map, const void* base, uint64_t atoms) {
  static EncodeTiledFn enc = (EncodeTiledFn)mthost::driver_entry("cuTensorMapEncodeTiled");
  if (!enc) return fail("cuTensorMapEncodeTiled not available");
  if ((uintptr_t)base & 15) return fail("scale tensors must be 16-byte aligned");
  cuuint64_t dims[2] = {128, atoms};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled (scales) failed: CUresult " + std::to_string((int)r));
  return 0;
}

int check_shape(int M, int N, int K, int nranks) {
  if (M <= 0 || N <= 0 || K <= 0) return fail("bad GEMM shape");
  if (M % (kBM * nranks) || N % kBN || K % kBK)
    return fail("GEMM shape: M must be a multiple of 128 x ranks, N of 256, K of 64");
  return 0;
}

int sm_count(int device) {
  int n = 148;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
  return n;
}

}  // namespace

namespace mthost {
int make_bf16_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
  return make_map(map, base, rows, K, box_rows);
}
}  // namespace mthost

// Row blocks per group of the plain GEMM's tile order.  Row-major order streams the whole of B through the
// L2 once per wave of CTAs; when B does not fit beside A's rows (large N x K) a grouped order keeps a wave's
// operands resident.  MINTCCL_GEMM_RASTER overrides (for tuning).
static int raster_for(int /*M*/, int N, int K, int elem_bytes) {
  if (const char* e = getenv("MINTCCL_GEMM_RASTER")) return atoi(e);
  const double b_bytes = (double)N * K * elem_bytes;
  return b_bytes > 48e6 ? 16 : 1;
}

// GEMMs run on CTA pairs (one 256 x 256 tile per cluster of two CTAs, gemm_tc2.cu) when the rows (of the
// problem for the plain GEMM, of one rank for the fused kernels) are a multiple of 256; otherwise, and with
// MINTCCL_GEMM_PAIR=0, on the single-CTA kernels of gemm_tc.cu.
static int g_pair_mode = -1;
static bool use_pair(int M) {
  if (g_pair_mode < 0) {
    const char* e = getenv("MINTCCL_GEMM_PAIR");
    g_pair_mode = e ? atoi(e) : kPairDefault;
  }
  return g_pair_mode != 0 && M % 256 == 0;
}

// Tile width of a bf16 pair GEMM over `row_tiles` 256-row blocks on `nclusters` clusters: 224 columns when N
// allows it and the waves of narrower tiles add up to less work than the waves of 256-column tiles
// (MINTCCL_GEMM_BN=256 / 224 forces one).
static int pick_bn(int row_tiles, int N, int nclusters, bool fp8) {
  if (fp8 || N % 224 || nclusters < 1) return 256;
  if (const char* e = getenv("MINTCCL_GEMM_BN")) {
    const int v = atoi(e);
    if (v == 224 || v == 256) return v;
  }
  const long w256 = (long)((row_tiles * (N / 256) + nclusters - 1) / nclusters) * 256;
  const long w224 = (long)((row_tiles * (N / 224) + nclusters - 1) / nclusters) * 224;
  return w224 < w256 ? 224 : 256;
}

static int gemm_pair(void* stream, const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N,
                     int K, int ldc, int nctas, bool fp8) {
  int dev = 0;
  cudaGetDevice(&dev);
  int ncl = (nctas > 0 ? nctas : sm_count(dev)) / 2;
  {
    const int fit = mt::gemm_pair_max_clusters(mt::MODE_PLAIN, fp8);
    if (fit > 0 && ncl > fit) ncl = fit;
  }
  const int bn = pick_bn(M / 256, N, ncl, fp8);
  mt::GemmMaps maps;
  mt::PairSfMaps sf;
  memset(&maps, 0, sizeof(maps));
  memset(&sf, 0, sizeof(sf));
  if (make_map(&maps.a[0], A, M, K, 128, fp8) || make_map(&maps.b[0], B, N, K, bn / 2, fp8)) return -1;
  maps.a2[0] = maps.a[0];
  if (fp8) {
    if (make_sf_map(&sf.sfa[0], sfa, (uint64_t)(M / 128) * (K / 128)) ||
        make_sf_map(&sf.sfb[0], sfb, (uint64_t)(N / 128) * (K / 128)))
      return -1;
  }
  mt::GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.c[0] = C;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.nranks = 1;
  a.raster = raster_for(M, N, K, fp8 ? 1 : 2) / 2;
  a.timeout_ns = 4000000000ull;
  const int tiles = (M / 256) * (N / bn);
  int nclusters = (nctas > 0 ? nctas : sm_count(dev)) / 2;
  if (nclusters > tiles) nclusters = tiles;
  if (nclusters < 1) nclusters = 1;
  cudaError_t e = mt::launch_gemm_pair(mt::MODE_PLAIN, maps, sf, a, nclusters, 1, (cudaStream_t)stream, fp8, bn);
  if (e != cudaSuccess) return fail(std::string("pair gemm launch: ") + cudaGetErrorString(e));
  mthost::stat_add(fp8 ? mthost::ST_GEMM_MXFP8 : mthost::ST_GEMM, (uint64_t)(2.0 * M * N * K));
  return 0;
}

extern "C" {

// 1 after a bounded wait of the CTA-pair GEMM expired (the result of that call is then invalid), 0 otherwise.
int mt_gemm_pair_error(void) { return mt::gemm_pair_error(); }
// 1: plain GEMMs use CTA pairs where the shape allows, 0: single-CTA kernel, -1: back to the environment / default.
void mt_gemm_set_pair(int mode) { g_pair_mode = mode; }

// C[M, ldc] = A[M, K] * B[N, K]^T in bf16 with fp32 accumulation, on the current device.
int mt_gemm(void* stream, const void* A, const void* B, void* C, int M, int N, int K, int ldc, int nctas) {
  if (check_shape(M, N, K, 1)) return -1;
  if (ldc < N || ldc % 8 || ((uintptr_t)C & 15)) return fail("C must be 16-byte aligned with ldc >= N, ldc % 8 == 0");
  if (use_pair(M)) return gemm_pair(stream, A, nullptr, B, nullptr, C, M, N, K, ldc, nctas, false);
  int dev = 0;
  cudaGetDevice(&dev);
  mt::GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  if (make_map(&maps.a[0], A, M, K, kBM) || make_map(&maps.b[0], B, N, K, kBN)) return -1;
  maps.a2[0] = maps.a[0];
  mt::GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.c[0] = C;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.nranks = 1;
  a.raster = raster_for(M, N, K, 2);
  a.timeout_ns = 4000000000ull;
  const int tiles = (M / kBM) * (N / kBN);
  int grid = nctas > 0 ? nctas : sm_count(dev);
  if (grid > tiles) grid = tiles;
  cudaError_t e = mt::launch_gemm_tc(mt::MODE_PLAIN, maps, a, grid, 1, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("gemm launch: ") + cudaGetErrorString(e));
  mthost::stat_add(mthost::ST_GEMM, (uint64_t)(2.0 * M * N * K));
  return 0;
}

// C[M, ldc] (bf16) = (A * SFA)[M, K] * (B * SFB)[N, K]^T for MXFP8 operands: e4m3 payload, ue8m0 scales per 32
// elements along K.  The scales are given in the tiled layout the tensor core reads: [rows / 128][K / 128][512]
// with byte (r % 32) * 16 + ((r % 128) / 32) * 4 + (k / 32) % 4 for row r and element k
// (mintccl_b200.ops.mxfp8.tile_scales builds it).  K must be a multiple of 128.
int mt_gemm_mxfp8(void* stream, const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N,
                  int K, int ldc, int nctas) {
  if (check_shape(M, N, K, 1) || K % 128) return fail("MXFP8 GEMM: M multiple of 128, N of 256, K of 128");
  if (ldc < N || ldc % 8 || ((uintptr_t)C & 15)) return fail("C must be 16-byte aligned with ldc >= N, ldc % 8 == 0");
  if (((uintptr_t)sfa | (uintptr_t)sfb) & 15) return fail("scale tensors must be 16-byte aligned");
  if (use_pair(M)) return gemm_pair(stream, A, sfa, B, sfb, C, M, N, K, ldc, nctas, true);
  int dev = 0;
  cudaGetDevice(&dev);
  mt::GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  if (make_map(&maps.a[0], A, M, K, kBM, true) || make_map(&maps.b[0], B, N, K, kBN, true)) return -1;
  maps.a2[0] = maps.a[0];
  mt::GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.c[0] = C;
  a.sfa[0] = sfa;
  a.sfb[0] = sfb;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = ldc;
  a.nranks = 1;
  a.raster = raster_for(M, N, K, 1);
  a.timeout_ns = 4000000000ull;
  const int tiles = (M / kBM) * (N / kBN);
  int grid = nctas > 0 ? nctas : sm_count(dev);
  if (grid > tiles) grid = tiles;
  cudaError_t e = mt::launch_gemm_tc(mt::MODE_PLAIN, maps, a, grid, 1, (cudaStream_t)stream, true);
  if (e != cudaSuccess) return fail(std::string("mxfp8 gemm launch: ") + cudaGetErrorString(e));
  mthost::stat_add(mthost::ST_GEMM_MXFP8, (uint64_t)(2.0 * M * N * K));
  return 0;
}

static int fused_common(MtComm* c, mt::GemmArgs& a, int M, int N, int K, uint64_t flags_off, uint64_t epoch) {
  if (!c || !c->d_comms) return fail("communicator is not finalized");
  if (check_shape(M, N, K, c->nranks)) return -1;
  memset(&a, 0, sizeof(a));
  a.M = M;
  a.N = N;
  a.K = K;
  a.nranks = c->nranks;
  a.comms = c->d_comms;
  a.flags_off = flags_off;
  a.epoch = epoch;
  a.timeout_ns = c->timeout_ns;
  for (int lr = 0; lr < c->nlocal; ++lr) {
    const int r = c->emulated ? lr : c->rank;
    a.rank[lr] = r;
    a.status[lr] = c->heap[lr][r] + c->L.status_off;
  }
  return 0;
}

// C[M, ldc] = allgather(a_shard)[M, K] * B[N, K]^T.  `gather_off`: symmetric buffer of M * K bf16;
// `flags_off`: symmetric u64 counters [ranks][M / ranks / 128], zero before the first call; `epoch`: 1 on the
// first call on these counters, then 2, 3, ...; `ncomm` must not change between calls on the same counters.
static int ag_gemm_impl(MtComm* c, void* stream, const void* const* a_shard, const void* const* B, void* const* C,
                        uint64_t gather_off, uint64_t flags_off, uint64_t epoch, int M, int N, int K, int ldc, int ncomm,
                        int nctas, int comm_mode, uint64_t shard_off, int comm_split, bool fp8, const void* const* sfa,
                        const void* const* sfb) {
  mt::GemmArgs a;
  if (fp8 && K % 128) return fail("MXFP8: K must be a multiple of 128");
  if (fused_common(c, a, M, N, K, flags_off, epoch)) return -1;
  if (ldc < N || ldc % 8) return fail("ldc must be >= N and a multiple of 8");
  const int n = c->nranks;
  if (n == 1) ncomm = 0;
  else if (ncomm < 1 || ncomm > 64) return fail("ncomm out of range");
  int grid = nctas > 0 ? nctas : sm_count(c->device);
  if (c->emulated && grid * c->nlocal > sm_count(c->device)) grid = sm_count(c->device) / c->nlocal;
  if (grid <= ncomm) return fail("not enough CTAs for the requested comm CTAs");
  if (ncomm > MT_MAX_BAR_SLOTS) return fail("too many comm CTAs");
  a.ldc = ldc;
  a.ncomm = ncomm;
  a.gather_off = gather_off;
  a.comm_mode = comm_mode;
  if (n > 1 && (comm_split < 1 || comm_split > ncomm)) return fail("comm_split must be in [1, ncomm]");
  a.comm_split = n > 1 ? comm_split : 1;
  a.shard_off = shard_off;
  if (comm_mode < 0 || comm_mode > 3) return fail("comm_mode must be 0, 1, 2 or 3");
  mt::GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  for (int lr = 0; lr < c->nlocal; ++lr) {
    const int r = a.rank[lr];
    a.c[lr] = C[lr];
    a.a_local[lr] = a_shard[lr];
    a.flags_local[lr] = c->heap[lr][r] + flags_off;
    if (make_map(&maps.a[lr], c->heap[lr][r] + gather_off, M, K, kBM, fp8) || make_map(&maps.b[lr], B[lr], N, K, kBN, fp8) ||
        make_map(&maps.a2[lr], a_shard[lr], M / n, K, kBM, fp8))
      return -1;
    if ((uintptr_t)C[lr] & 15) return fail("C must be 16-byte aligned");
    if (fp8) {
      a.sfa[lr] = sfa[lr];
      a.sfb[lr] = sfb[lr];
    }
  }
  if (use_pair(M / n) && comm_mode != 2) {
    // CTA pairs: 256-row tiles inside one owner's rows, B split between the two CTAs, comm CTAs in whole clusters
    mt::PairSfMaps sf;
    memset(&sf, 0, sizeof(sf));
    a.ncomm = (ncomm + 1) & ~1;
    if (a.comm_split > 1 && a.ncomm % a.comm_split) return fail("comm_split must divide the (even) number of comm CTAs");
    const int nclusters = (grid - a.ncomm) / 2;
    if (nclusters < 1) return fail("not enough CTAs for the requested comm CTAs");
    const int bn = pick_bn(M / 256, N, nclusters, fp8);
    for (int lr = 0; lr < c->nlocal; ++lr) {
      if (make_map(&maps.b[lr], B[lr], N, K, bn / 2, fp8)) return -1;
      if (fp8 && (make_sf_map(&sf.sfa[lr], sfa[lr], (uint64_t)(M / 128) * (K / 128)) ||
                  make_sf_map(&sf.sfb[lr], sfb[lr], (uint64_t)(N / 128) * (K / 128))))
        return -1;
    }
    cudaError_t e2 = mt::launch_gemm_pair(mt::MODE_AG_GEMM, maps, sf, a, nclusters, c->nlocal, (cudaStream_t)stream, fp8, bn);
    if (e2 != cudaSuccess) return fail(std::string("pair ag_gemm launch: ") + cudaGetErrorString(e2));
    mthost::stat_add(mthost::ST_AG_GEMM, (uint64_t)(2.0 * M * N * K));
    return 0;
  }
  cudaError_t e = mt::launch_gemm_tc(mt::MODE_AG_GEMM, maps, a, grid, c->nlocal, (cudaStream_t)stream, fp8);
  if (e != cudaSuccess) return fail(std::string("ag_gemm launch: ") + cudaGetErrorString(e));
  mthost::stat_add(mthost::ST_AG_GEMM, (uint64_t)(2.0 * M * N * K));
  return 0;
}

int mt_ag_gemm(MtComm* c, void* stream, const void* const* a_shard, const void* const* B, void* const* C,
               uint64_t gather_off, uint64_t flags_off, uint64_t epoch, int M, int N, int K, int ldc, int ncomm,
               int nctas, int comm_mode, uint64_t shard_off, int comm_split) {
  return ag_gemm_impl(c, stream, a_shard, B, C, gather_off, flags_off, epoch, M, N, K, ldc, ncomm, nctas, comm_mode,
                      shard_off, comm_split, false, nullptr, nullptr);
}
// MXFP8 variant: payloads are e4m3 bytes; `sfa` is the tiled scale tensor of the GATHERED A (every rank must
// hold all of it before the call, e.g. through an all-gather of the small scale tensors), `sfb` that of B.
int mt_ag_gemm_mxfp8(MtComm* c, void* stream, const void* const* a_shard, const void* const* sfa, const void* const* B,
                     const void* const* sfb, void* const* C, uint64_t gather_off, uint64_t flags_off, uint64_t epoch,
                     int M, int N, int K, int ldc, int ncomm, int nctas) {
  return ag_gemm_impl(c, stream, a_shard, B, C, gather_off, flags_off, epoch, M, N, K, ldc, ncomm, nctas, 0, 0, 1, true,
                      sfa, sfb);
}

// out[M / ranks, N] = reduce_scatter over rows of (A[M, K] * B[N, K]^T), K being this rank's slice of the
// contraction.  `stage_off`: symmetric buffer of 2 * ranks * (M / ranks) * N bf16 partial tiles.  Calls alternate
// between its halves (by the parity of `epoch`): a rank that has finished call e may already write partial tiles
// of call e + 1 into a peer whose reducers still read those of call e; it cannot reach call e + 2 before that
// peer has finished call e, because call e + 1 needs the peer's partial tiles of call e + 1.
// `flags_off`: symmetric u64 counters [ranks][M / ranks / 128][N / 256] followed by two ticket words, all zero
// before the first call.  `nred`: CTAs that only reduce (the others join them when their tiles are done).
static int gemm_rs_impl(MtComm* c, void* stream, const void* const* A, const void* const* B, void* const* out,
                        uint64_t stage_off, uint64_t flags_off, uint64_t epoch, int M, int N, int K, int nred, int nctas,
                        bool fp8, const void* const* sfa, const void* const* sfb) {
  mt::GemmArgs a;
  if (fp8 && K % 128) return fail("MXFP8: K must be a multiple of 128");
  if (fused_common(c, a, M, N, K, flags_off, epoch)) return -1;
  int grid = nctas > 0 ? nctas : sm_count(c->device);
  if (c->emulated && grid * c->nlocal > sm_count(c->device)) grid = sm_count(c->device) / c->nlocal;
  if (nred < 0 || nred >= grid) return fail("nred out of range");
  a.ncomm = nred;
  a.ldc = N;
  a.stage_off = stage_off + (epoch & 1) * (uint64_t)M * N * 2;
  mt::GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  for (int lr = 0; lr < c->nlocal; ++lr) {
    a.c[lr] = out[lr];
    if (make_map(&maps.a[lr], A[lr], M, K, kBM, fp8) || make_map(&maps.b[lr], B[lr], N, K, kBN, fp8)) return -1;
    maps.a2[lr] = maps.a[lr];
    if ((uintptr_t)out[lr] & 15) return fail("out must be 16-byte aligned");
    if (fp8) {
      a.sfa[lr] = sfa[lr];
      a.sfb[lr] = sfb[lr];
    }
  }
  if (use_pair(M / c->nranks)) {
    mt::PairSfMaps sf;
    memset(&sf, 0, sizeof(sf));
    for (int lr = 0; lr < c->nlocal; ++lr) {
      if (make_map(&maps.b[lr], B[lr], N, K, 128, fp8)) return -1;
      if (fp8 && (make_sf_map(&sf.sfa[lr], sfa[lr], (uint64_t)(M / 128) * (K / 128)) ||
                  make_sf_map(&sf.sfb[lr], sfb[lr], (uint64_t)(N / 128) * (K / 128))))
        return -1;
    }
    a.ncomm = (nred + 1) & ~1;
    const int nclusters = (grid - a.ncomm) / 2;
    if (nclusters < 1) return fail("nred out of range");
    cudaError_t e2 = mt::launch_gemm_pair(mt::MODE_GEMM_RS, maps, sf, a, nclusters, c->nlocal, (cudaStream_t)stream, fp8);
    if (e2 != cudaSuccess) return fail(std::string("pair gemm_rs launch: ") + cudaGetErrorString(e2));
    mthost::stat_add(mthost::ST_GEMM_RS, (uint64_t)(2.0 * M * N * K));
    return 0;
  }
  cudaError_t e = mt::launch_gemm_tc(mt::MODE_GEMM_RS, maps, a, grid, c->nlocal, (cudaStream_t)stream, fp8);
  if (e != cudaSuccess) return fail(std::string("gemm_rs launch: ") + cudaGetErrorString(e));
  mthost::stat_add(mthost::ST_GEMM_RS, (uint64_t)(2.0 * M * N * K));
  return 0;
}

int mt_gemm_rs(MtComm* c, void* stream, const void* const* A, const void* const* B, void* const* out,
               uint64_t stage_off, uint64_t flags_off, uint64_t epoch, int M, int N, int K, int nred, int nctas) {
  return gemm_rs_impl(c, stream, A, B, out, stage_off, flags_off, epoch, M, N, K, nred, nctas, false, nullptr, nullptr);
}
int mt_gemm_rs_mxfp8(MtComm* c, void* stream, const void* const* A, const void* const* sfa, const void* const* B,
                     const void* const* sfb, void* const* out, uint64_t stage_off, uint64_t flags_off, uint64_t epoch,
                     int M, int N, int K, int nred, int nctas) {
  return gemm_rs_impl(c, stream, A, B, out, stage_off, flags_off, epoch, M, N, K, nred, nctas, true, sfa, sfb);
}

// Sum of MXFP8 tensors (e4m3 payload + ue8m0 scale per 32 elements) over all ranks.  op 0: all-reduce into
// (data_out_off, scale_out_off) of every rank; op 1: reduce-scatter, shard `rank` into the local outputs.
int mt_mxfp8_reduce(MtComm* c, void* stream, int op, uint64_t data_in_off, uint64_t scale_in_off,
                    uint64_t data_out_off, uint64_t scale_out_off, void* const* data_out, void* const* scale_out,
                    uint64_t nelems, int nctas) {
  if (!c || !c->d_comms) return fail("communicator is not finalized");
  if (nelems % 32) return fail("MXFP8 tensors hold whole blocks of 32 elements");
  const uint64_t nblocks = nelems / 32;
  if (op == mt::MX_REDUCESCATTER && nblocks % c->nranks) return fail("blocks must divide evenly over the ranks");
  if ((data_in_off | data_out_off) & 15) return fail("MXFP8 payloads must be 16-byte aligned");
  if (nctas < 1 || nctas > 148) return fail("nctas out of range");
  if (c->emulated && nctas * c->nlocal > 148) nctas = 148 / c->nlocal;
  mt::Mxfp8Args a;
  memset(&a, 0, sizeof(a));
  a.data_in_off = data_in_off;
  a.scale_in_off = scale_in_off;
  a.data_out_off = data_out_off;
  a.scale_out_off = scale_out_off;
  a.nblocks = nblocks;
  a.op = op;
  for (int lr = 0; lr < c->nlocal; ++lr) {
    a.data_out[lr] = data_out ? data_out[lr] : nullptr;
    a.scale_out[lr] = scale_out ? scale_out[lr] : nullptr;
  }
  cudaError_t e = mt::launch_mxfp8(c->d_comms, a, nctas, c->nlocal, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("mxfp8 launch: ") + cudaGetErrorString(e));
  mthost::stat_add(mthost::ST_MXFP8_REDUCE, nelems);
  return 0;
}

}  // extern "C"
