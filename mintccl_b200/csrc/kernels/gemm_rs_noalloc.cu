// Single-rank GEMM -> reduce-scatter with its scratch memory in a file-scope device array, for callers
// that cannot allocate (see gemm_rs_noalloc.h).  The kernel is the regular one; only where its scratch
// lives differs: the "heap" it is given is the array below.
#include "gemm_rs_noalloc.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include <mutex>
#include <string>

#include "../device/layout.h"
#include "../host/comm_internal.h"
#include "gemm_tc.h"

namespace {

// Layout of the scratch array (offsets in bytes).
constexpr uint64_t kCommOff = 0;          // MtDevComm read by the kernel
constexpr uint64_t kStatusOff = 2048;     // MtStatus written by the kernel on a failed wait
constexpr uint64_t kFlagsOff = 4096;      // u64 arrival counters [M / 128][N / 256], then two ticket words
constexpr uint64_t kFlagsBytes = (MT_NOALLOC_MAX_M / 128) * (MT_NOALLOC_MAX_N / 256) * 8 + 16;  // + two ticket words
constexpr uint64_t kStageOff = 8192;      // bf16 partial tiles [M][N]
constexpr uint64_t kStageBytes = (uint64_t)MT_NOALLOC_MAX_M * MT_NOALLOC_MAX_N * 2;
constexpr uint64_t kScratchBytes = kStageOff + kStageBytes;
static_assert(kFlagsOff + kFlagsBytes <= kStageOff, "counters overlap the partial tiles");
static_assert(sizeof(MtDevComm) <= kStatusOff, "descriptor does not fit");

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_dev[kMaxDevices] = {};  // device address of g_scratch, per device

// Once per device, with that device current: resolve the array's device address and store the
// descriptor the kernel expects (a one-rank communicator whose heap is the array).
int setup(int dev, unsigned char** out) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_dev[dev]) {
    *out = g_scratch_dev[dev];
    return 0;
  }
  unsigned char* ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_scratch);
  if (e != cudaSuccess || !ptr) return mthost::fail(std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
  MtDevComm d;
  memset(&d, 0, sizeof(d));
  d.rank = 0;
  d.nranks = 1;
  d.ring_pos = 0;
  d.timeout_ns = 4000000000ull;
  d.heap[0] = ptr;
  d.L.status_off = kStatusOff;
  e = cudaMemcpy(ptr + kCommOff, &d, sizeof(d), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemset(ptr + kStatusOff, 0, sizeof(MtStatus));
  if (e != cudaSuccess) return mthost::fail(std::string("scratch set-up: ") + cudaGetErrorString(e));
  g_scratch_dev[dev] = ptr;
  *out = ptr;
  return 0;
}

}  // namespace

extern "C" int mt_gemm_rs_single_noalloc(void* stream, const void* A, const void* B, void* out, int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 256 || K % 64)
    return mthost::fail("mt_gemm_rs_single_noalloc: M must be a multiple of 128, N of 256, K of 64");
  if (M > MT_NOALLOC_MAX_M || N > MT_NOALLOC_MAX_N)
    return mthost::fail("mt_gemm_rs_single_noalloc: problem exceeds the built-in scratch (M <= " +
                        std::to_string(MT_NOALLOC_MAX_M) + ", N <= " + std::to_string(MT_NOALLOC_MAX_N) + "), got M=" +
                        std::to_string(M) + " N=" + std::to_string(N));
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)out) & 15)
    return mthost::fail("mt_gemm_rs_single_noalloc: pointers must be 16-byte aligned");
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return mthost::fail("mt_gemm_rs_single_noalloc: no usable current device");
  unsigned char* scratch = nullptr;
  if (setup(dev, &scratch)) return -1;

  mt::GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  if (mthost::make_bf16_map(&maps.a[0], A, M, K, 128) || mthost::make_bf16_map(&maps.b[0], B, N, K, 256)) return -1;
  maps.a2[0] = maps.a[0];
  mt::GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.c[0] = out;
  a.status[0] = scratch + kStatusOff;
  a.comms = (const MtDevComm*)(scratch + kCommOff);
  a.rank[0] = 0;
  a.M = M;
  a.N = N;
  a.K = K;
  a.ldc = N;
  a.nranks = 1;
  a.flags_off = kFlagsOff;
  a.stage_off = kStageOff;
  a.epoch = 1;  // the counters are cleared below, so every call is "the first"
  a.timeout_ns = 4000000000ull;
  // the array keeps the previous call's counters: they must start at zero
  cudaError_t e = cudaMemsetAsync(scratch + kFlagsOff, 0, kFlagsBytes, (cudaStream_t)stream);
  if (e != cudaSuccess) return mthost::fail(std::string("clearing the counters: ") + cudaGetErrorString(e));
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  e = mt::launch_gemm_tc(mt::MODE_GEMM_RS, maps, a, sms, 1, (cudaStream_t)stream);
  if (e != cudaSuccess) return mthost::fail(std::string("mt_gemm_rs_single_noalloc launch: ") + cudaGetErrorString(e));
  return 0;
}

// A wait inside the kernel that ran out of time leaves its record in the scratch array, not in any
// communicator: this reads it back (and clears it on request).  Synchronises the device.
extern "C" int mt_gemm_rs_single_noalloc_status(MtStatus* out, int clear) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return mthost::fail("mt_gemm_rs_single_noalloc_status: no usable current device");
  unsigned char* scratch = nullptr;
  if (setup(dev, &scratch)) return -1;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess && out) e = cudaMemcpy(out, scratch + kStatusOff, sizeof(MtStatus), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && clear) e = cudaMemset(scratch + kStatusOff, 0, sizeof(MtStatus));
  if (e != cudaSuccess) return mthost::fail(std::string("mt_gemm_rs_single_noalloc_status: ") + cudaGetErrorString(e));
  return 0;
}
