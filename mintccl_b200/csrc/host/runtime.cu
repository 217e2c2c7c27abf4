// Host runtime: symmetric heap (cuMem VMM with POSIX-fd export, or cudaMalloc + cudaIpc), peer
// mapping, NVLS multicast binding, device descriptors, launch wrappers, status read-back.
//
// Stands where the reference has `set_gpu`, `send_ptr` and `recv_ptr` (common.py:10-38).  Differences:
// everything is mapped once per communicator instead of once per call; an ordinary allocation is
// registered by the handle of its *containing* allocation plus the offset inside it (the reference
// sends the handle of the block and drops the offset, common.py:24-26); handles are cached and closed.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../device/sched.h"
#include "../kernels/direct_engine.cuh"
#include "../kernels/launch.h"
#include "../kernels/p2p_engine.cuh"
#include "../kernels/ring_engine.cuh"
#include "../mintccl.h"
#include "comm_internal.h"

namespace {

thread_local std::string g_err;
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_stat_calls[mthost::ST_COUNT], g_stat_work[mthost::ST_COUNT];
const char* const g_stat_names[mthost::ST_COUNT] = {"ring_simple", "ring_ll128", "direct", "nvls", "ll_oneshot", "p2p",
                                                     "local_copy", "gemm", "gemm_mxfp8", "ag_gemm", "gemm_rs", "mxfp8_reduce"};

int fail(const std::string& m) {
  g_err = m;
  return -1;
}
#define CUDA_OK(expr)                                                                    \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) return fail(std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

// Driver entry points are looked up through the runtime so that the library loads on machines
// without a driver (the CPU-only parts stay usable there).
template <class F>
F drv(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return (F)fn;
}
#define DRV(name) auto p_##name = drv<decltype(&name)>(#name); if (!p_##name) return fail("driver entry point " #name " not found")
#define CU_OK(expr)                                                         \
  do {                                                                      \
    CUresult _r = (expr);                                                   \
    if (_r != CUDA_SUCCESS) return fail(std::string(#expr) + " failed: CUresult " + std::to_string((int)_r)); \
  } while (0)

}  // namespace

namespace mthost {
int fail(const std::string& m) { return ::fail(m); }
void stat_add(int kind, uint64_t work) {
  if (kind < 0 || kind >= ST_COUNT) return;
  g_stat_calls[kind].fetch_add(1, std::memory_order_relaxed);
  g_stat_work[kind].fetch_add(work, std::memory_order_relaxed);
}
void* driver_entry(const char* name) { return (void*)drv<void*>(name); }
}  // namespace mthost

namespace mt {
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
cudaError_t launch_any(const void* fn, dim3 grid, dim3 block, void** args, cudaStream_t s, bool cooperative,
                       size_t dyn_smem) {
  count_launch();
  if (cooperative) return cudaLaunchCooperativeKernel(fn, grid, block, args, dyn_smem, s);
  return cudaLaunchKernel(fn, grid, block, args, dyn_smem, s);
}
}  // namespace mt

static uint64_t granularity_for(int device, bool want_mc, int nranks) {
  auto p_gran = drv<decltype(&cuMemGetAllocationGranularity)>("cuMemGetAllocationGranularity");
  uint64_t g = 2ull << 20;
  if (p_gran) {
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gg = 0;
    if (p_gran(&gg, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && gg) g = gg;
  }
  if (want_mc) {
    auto p_mcg = drv<decltype(&cuMulticastGetGranularity)>("cuMulticastGetGranularity");
    if (p_mcg) {
      CUmulticastObjectProp mp{};
      mp.numDevices = nranks;
      mp.size = 1ull << 30;
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      size_t gg = 0;
      if (p_mcg(&gg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && gg > g) g = gg;
    }
  }
  return g;
}

static int vmm_map(MtComm* c, CUmemGenericAllocationHandle h, uint8_t** out) {
  DRV(cuMemAddressReserve);
  DRV(cuMemMap);
  DRV(cuMemSetAccess);
  CUdeviceptr va = 0;
  CU_OK(p_cuMemAddressReserve(&va, c->heap_bytes, 0, 0, 0));
  CU_OK(p_cuMemMap(va, c->heap_bytes, 0, h, 0));
  CUmemAccessDesc ad{};
  ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  ad.location.id = c->device;
  ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CU_OK(p_cuMemSetAccess(va, c->heap_bytes, &ad, 1));
  *out = (uint8_t*)va;
  return 0;
}

static void fill_layout(MtComm* c, const MtConfig* cfg, int nranks) {
  c->cfg = *cfg;
  c->L = mt_make_layout(nranks, cfg->nchannels, cfg->simple_slot_bytes, cfg->simple_slots, cfg->ll128_slot_bytes,
                        cfg->ll128_slots, cfg->ll_bytes, cfg->scratch_bytes, cfg->heap_bytes);
  c->timeout_ns = cfg->timeout_ms * 1000000ull;
}

extern "C" {

const char* mt_last_error(void) { return g_err.c_str(); }
int mt_version(void) { return 100; }
uint64_t mt_launch_count(void) { return g_launches.load(); }
void mt_reset_launch_count(void) { g_launches.store(0); }

int mt_stats_count(void) { return mthost::ST_COUNT; }
const char* mt_stats_name(int kind) { return kind >= 0 && kind < mthost::ST_COUNT ? g_stat_names[kind] : ""; }
int mt_stats_get(int kind, uint64_t* calls, uint64_t* work) {
  if (kind < 0 || kind >= mthost::ST_COUNT) return -1;
  if (calls) *calls = g_stat_calls[kind].load();
  if (work) *work = g_stat_work[kind].load();
  return 0;
}
void mt_stats_reset(void) {
  for (int i = 0; i < mthost::ST_COUNT; ++i) {
    g_stat_calls[i].store(0);
    g_stat_work[i].store(0);
  }
}

static int check_cfg(const MtConfig* cfg, int nranks) {
  if (nranks < 1 || nranks > MT_MAX_RANKS) return fail("nranks must be in [1, 8]");
  if (cfg->nchannels < 1 || cfg->nchannels > MT_MAX_CHANNELS) return fail("nchannels must be in [1, 96]");
  if (cfg->simple_slots < 1 || cfg->ll128_slots < 1) return fail("need at least one FIFO slot");
  if (cfg->simple_slot_bytes % 128 || cfg->ll128_slot_bytes % MT_LL128_WARP_WIRE || cfg->ll_bytes % MT_LL128_WARP_WIRE)
    return fail("slot sizes must be multiples of 128 (Simple) / 2048 (LL128, one-shot)");
  return 0;
}

uint64_t mt_layout_user_off(int nranks, const MtConfig* cfg) {
  return mt_make_layout(nranks, cfg->nchannels, cfg->simple_slot_bytes, cfg->simple_slots, cfg->ll128_slot_bytes,
                        cfg->ll128_slots, cfg->ll_bytes, cfg->scratch_bytes, cfg->heap_bytes)
      .user_off;
}

MtComm* mt_comm_create(int rank, int nranks, int device, const MtConfig* cfg) {
  if (check_cfg(cfg, nranks)) return nullptr;
  if (cudaSetDevice(device) != cudaSuccess) {
    fail("cudaSetDevice failed");
    return nullptr;
  }
  cudaFree(0);
  MtComm* c = new MtComm();
  c->rank = rank;
  c->nranks = nranks;
  c->device = device;
  c->heap_kind = cfg->heap_kind;
  fill_layout(c, cfg, nranks);
  if (c->L.user_off > cfg->heap_bytes) {
    fail("heap_bytes smaller than the control region (" + std::to_string(c->L.user_off) + " bytes)");
    delete c;
    return nullptr;
  }
  auto bail = [&](const char* what) -> MtComm* {
    if (g_err.empty()) fail(what);
    delete c;
    return nullptr;
  };
  if (c->heap_kind == 0) {
    auto p_create = drv<decltype(&cuMemCreate)>("cuMemCreate");
    if (!p_create) return bail("cuMemCreate not available");
    const uint64_t g = granularity_for(device, true, nranks);
    c->heap_bytes = mt_round_up(cfg->heap_bytes, g);
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUresult r = p_create(&c->local_handle, c->heap_bytes, &prop, 0);
    if (r != CUDA_SUCCESS) {
      fail("cuMemCreate failed: CUresult " + std::to_string((int)r));
      return bail("cuMemCreate");
    }
    c->own_vmm = true;
    if (vmm_map(c, c->local_handle, &c->heap[0][rank])) return bail("map");
  } else {
    c->heap_bytes = mt_round_up(cfg->heap_bytes, 2ull << 20);
    void* p = nullptr;
    if (cudaMalloc(&p, c->heap_bytes) != cudaSuccess) return bail("cudaMalloc of the heap failed");
    c->heap[0][rank] = (uint8_t*)p;
  }
  c->L.heap_bytes = c->heap_bytes;
  if (cudaMemset(c->heap[0][rank], 0, c->L.user_off) != cudaSuccess) return bail("cudaMemset failed");
  cudaDeviceSynchronize();
  return c;
}

MtComm* mt_comm_create_emulated(int nranks, int device, const MtConfig* cfg) {
  if (check_cfg(cfg, nranks)) return nullptr;
  if (cudaSetDevice(device) != cudaSuccess) {
    fail("cudaSetDevice failed");
    return nullptr;
  }
  MtComm* c = new MtComm();
  c->emulated = true;
  c->nranks = nranks;
  c->nlocal = nranks;
  c->device = device;
  c->heap_kind = 1;
  fill_layout(c, cfg, nranks);
  if (c->L.user_off > cfg->heap_bytes) {
    // the FIFOs and control words alone are larger than the heap: kernels would run off its end
    fail("heap_bytes smaller than the control region (" + std::to_string(c->L.user_off) + " bytes)");
    delete c;
    return nullptr;
  }
  c->heap_bytes = mt_round_up(cfg->heap_bytes, 2ull << 20);
  c->L.heap_bytes = c->heap_bytes;
  for (int r = 0; r < nranks; ++r) {
    void* p = nullptr;
    if (cudaMalloc(&p, c->heap_bytes) != cudaSuccess) {
      fail("cudaMalloc of an emulated heap failed");
      mt_comm_destroy(c);
      return nullptr;
    }
    c->emu_allocs.push_back(p);
    cudaMemset(p, 0, c->L.user_off);
  }
  for (int lr = 0; lr < nranks; ++lr)
    for (int p = 0; p < nranks; ++p) c->heap[lr][p] = (uint8_t*)c->emu_allocs[p];
  cudaDeviceSynchronize();
  return c;
}

void mt_comm_destroy(MtComm* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  mt_reg_stop(c);
  auto p_unmap = drv<decltype(&cuMemUnmap)>("cuMemUnmap");
  auto p_release = drv<decltype(&cuMemRelease)>("cuMemRelease");
  auto p_free = drv<decltype(&cuMemAddressFree)>("cuMemAddressFree");
  if (c->d_comms) cudaFree(c->d_comms);
  if (c->emulated) {
    for (void* p : c->emu_allocs) cudaFree(p);
  } else if (c->heap_kind == 0 && p_unmap && p_release && p_free) {
    if (c->mc) {
      p_unmap((CUdeviceptr)c->mc, c->heap_bytes);
      p_free((CUdeviceptr)c->mc, c->heap_bytes);
    }
    if (c->mc_bound) {
      auto p_unbind = drv<decltype(&cuMulticastUnbind)>("cuMulticastUnbind");
      CUdevice dev;
      auto p_devget = drv<decltype(&cuDeviceGet)>("cuDeviceGet");
      if (p_unbind && p_devget && p_devget(&dev, c->device) == CUDA_SUCCESS) p_unbind(c->mc_handle, dev, 0, c->heap_bytes);
    }
    if (c->mc_have_handle) p_release(c->mc_handle);
    for (int p = 0; p < c->nranks; ++p) {
      if (p == c->rank || !c->peer_mapped[p]) continue;
      p_unmap((CUdeviceptr)c->heap[0][p], c->heap_bytes);
      p_free((CUdeviceptr)c->heap[0][p], c->heap_bytes);
      p_release(c->peer_handle[p]);
    }
    if (c->own_vmm) {
      p_unmap((CUdeviceptr)c->heap[0][c->rank], c->heap_bytes);
      p_free((CUdeviceptr)c->heap[0][c->rank], c->heap_bytes);
      p_release(c->local_handle);
    }
  } else if (c->heap_kind == 1) {
    for (int p = 0; p < c->nranks; ++p)
      if (p != c->rank && c->ipc_opened[p]) cudaIpcCloseMemHandle(c->ipc_opened[p]);
    if (c->heap[0][c->rank]) cudaFree(c->heap[0][c->rank]);
  }
  delete c;
}

int mt_comm_heap_kind(MtComm* c) { return c->heap_kind; }
int mt_comm_nlocal(MtComm* c) { return c->nlocal; }

int mt_comm_export_fd(MtComm* c) {
  if (c->heap_kind != 0 || c->emulated) return fail("heap is not a VMM allocation");
  DRV(cuMemExportToShareableHandle);
  int fd = -1;
  CU_OK(p_cuMemExportToShareableHandle(&fd, c->local_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  return fd;
}

int mt_comm_export_ipc(MtComm* c, unsigned char handle[64]) {
  if (c->heap_kind != 1 || c->emulated) return fail("heap is not a cudaMalloc allocation");
  cudaIpcMemHandle_t h;
  CUDA_OK(cudaIpcGetMemHandle(&h, c->heap[0][c->rank]));
  static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
  memcpy(handle, &h, 64);
  return 0;
}

int mt_comm_import_fd(MtComm* c, int peer, int fd) {
  if (peer < 0 || peer >= c->nranks || peer == c->rank) return fail("bad peer");
  DRV(cuMemImportFromShareableHandle);
  CU_OK(p_cuMemImportFromShareableHandle(&c->peer_handle[peer], (void*)(uintptr_t)fd,
                                         CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  if (vmm_map(c, c->peer_handle[peer], &c->heap[0][peer])) return -1;
  c->peer_mapped[peer] = true;
  return 0;
}

int mt_comm_import_ipc(MtComm* c, int peer, const unsigned char handle[64]) {
  if (peer < 0 || peer >= c->nranks || peer == c->rank) return fail("bad peer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  c->ipc_opened[peer] = p;
  c->heap[0][peer] = (uint8_t*)p;
  return 0;
}

int mt_comm_mc_supported(MtComm* c) {
  if (c->emulated || c->heap_kind != 0) return 0;
  int v = 0;
  auto p_attr = drv<decltype(&cuDeviceGetAttribute)>("cuDeviceGetAttribute");
  auto p_devget = drv<decltype(&cuDeviceGet)>("cuDeviceGet");
  CUdevice dev;
  if (!p_attr || !p_devget || p_devget(&dev, c->device) != CUDA_SUCCESS) return 0;
  if (p_attr(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return v;
}

int mt_comm_mc_create(MtComm* c) {
  DRV(cuMulticastCreate);
  DRV(cuMemExportToShareableHandle);
  CUmulticastObjectProp mp{};
  mp.numDevices = c->nranks;
  mp.size = c->heap_bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CU_OK(p_cuMulticastCreate(&c->mc_handle, &mp));
  c->mc_have_handle = true;
  int fd = -1;
  CU_OK(p_cuMemExportToShareableHandle(&fd, c->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  return fd;
}

int mt_comm_mc_import(MtComm* c, int fd) {
  DRV(cuMemImportFromShareableHandle);
  CU_OK(p_cuMemImportFromShareableHandle(&c->mc_handle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  c->mc_have_handle = true;
  return 0;
}

int mt_comm_mc_add_device(MtComm* c) {
  DRV(cuMulticastAddDevice);
  DRV(cuDeviceGet);
  CUdevice dev;
  CU_OK(p_cuDeviceGet(&dev, c->device));
  CU_OK(p_cuMulticastAddDevice(c->mc_handle, dev));
  return 0;
}

int mt_comm_mc_bind(MtComm* c) {
  DRV(cuMulticastBindMem);
  CU_OK(p_cuMulticastBindMem(c->mc_handle, 0, c->local_handle, 0, c->heap_bytes, 0));
  c->mc_bound = true;
  if (vmm_map(c, c->mc_handle, &c->mc)) return -1;
  return 0;
}

int mt_comm_set_ring(MtComm* c, const int* ring) {
  std::vector<int> seen(c->nranks, 0);
  for (int i = 0; i < c->nranks; ++i) {
    if (ring[i] < 0 || ring[i] >= c->nranks || seen[ring[i]]) return fail("ring must be a permutation of the ranks");
    seen[ring[i]] = 1;
    c->ring[i] = ring[i];
  }
  if (!c->d_comms) return 0;
  for (int lr = 0; lr < c->nlocal; ++lr) {
    MtDevComm& d = c->h_comms[lr];
    for (int i = 0; i < c->nranks; ++i) {
      d.ring[i] = c->ring[i];
      if (c->ring[i] == d.rank) d.ring_pos = i;
    }
  }
  CUDA_OK(cudaMemcpy(c->d_comms, c->h_comms, sizeof(MtDevComm) * c->nlocal, cudaMemcpyHostToDevice));
  return 0;
}

int mt_comm_finalize(MtComm* c, const int* ring) {
  cudaSetDevice(c->device);
  for (int lr = 0; lr < c->nlocal; ++lr) {
    const int r = c->emulated ? lr : c->rank;
    for (int p = 0; p < c->nranks; ++p)
      if (!c->heap[lr][p]) return fail("peer " + std::to_string(p) + " is not mapped");
    MtDevComm& d = c->h_comms[lr];
    memset(&d, 0, sizeof(d));
    d.rank = r;
    d.nranks = c->nranks;
    d.has_mc = c->mc != nullptr;
    d.timeout_ns = c->timeout_ns;
    for (int p = 0; p < c->nranks; ++p) d.heap[p] = c->heap[lr][p];
    d.mc = c->mc;
    d.L = c->L;
  }
  if (!c->d_comms) CUDA_OK(cudaMalloc(&c->d_comms, sizeof(MtDevComm) * MT_MAX_RANKS));
  if (mt_comm_set_ring(c, ring)) return -1;
  CUDA_OK(cudaMemcpy(c->d_comms, c->h_comms, sizeof(MtDevComm) * c->nlocal, cudaMemcpyHostToDevice));
  return 0;
}

int mt_comm_set_timeout_ms(MtComm* c, uint64_t ms) {
  c->timeout_ns = ms * 1000000ull;
  if (!c->d_comms) return 0;
  for (int lr = 0; lr < c->nlocal; ++lr) c->h_comms[lr].timeout_ns = c->timeout_ns;
  CUDA_OK(cudaMemcpy(c->d_comms, c->h_comms, sizeof(MtDevComm) * c->nlocal, cudaMemcpyHostToDevice));
  return 0;
}

void* mt_comm_heap_ptr(MtComm* c, int local_rank, int peer) {
  if (local_rank < 0 || local_rank >= c->nlocal || peer < 0 || peer >= c->nranks) return nullptr;
  return c->heap[local_rank][peer];
}
void* mt_comm_mc_ptr(MtComm* c) { return c->mc; }
int mt_comm_layout(MtComm* c, MtHeapLayout* out) {
  *out = c->L;
  return 0;
}

int mt_comm_status(MtComm* c, int local_rank, MtStatus* out) {
  if (local_rank < 0 || local_rank >= c->nlocal) return fail("bad local rank");
  cudaSetDevice(c->device);
  CUDA_OK(cudaDeviceSynchronize());
  const int r = c->emulated ? local_rank : c->rank;
  CUDA_OK(cudaMemcpy(out, c->heap[local_rank][r] + c->L.status_off, sizeof(MtStatus), cudaMemcpyDeviceToHost));
  return 0;
}

int mt_comm_clear_status(MtComm* c) {
  cudaSetDevice(c->device);
  CUDA_OK(cudaDeviceSynchronize());
  for (int lr = 0; lr < c->nlocal; ++lr) {
    const int r = c->emulated ? lr : c->rank;
    CUDA_OK(cudaMemset(c->heap[lr][r] + c->L.status_off, 0, sizeof(MtStatus)));
  }
  return 0;
}

// ---- registration of ordinary allocations ---------------------------------------------------------
// One mapping per CUDA IPC handle and process (the runtime refuses to open a handle twice), counted so that the
// users of a handle (Communicator.register, the registration services of several communicators) can close
// independently.
struct IpcMapping {
  void* base;
  int refs;
};
static std::mutex g_ipc_mu;
static std::map<std::string, IpcMapping> g_ipc_cache;

int mt_ipc_export(const void* ptr, unsigned char handle[64], uint64_t* offset, uint64_t* alloc_bytes) {
  DRV(cuMemGetAddressRange);
  CUdeviceptr base = 0;
  size_t size = 0;
  CU_OK(p_cuMemGetAddressRange(&base, &size, (CUdeviceptr)ptr));
  cudaIpcMemHandle_t h;
  CUDA_OK(cudaIpcGetMemHandle(&h, (void*)base));
  memcpy(handle, &h, 64);
  *offset = (uint64_t)((CUdeviceptr)ptr - base);
  *alloc_bytes = size;
  return 0;
}

void* mt_ipc_open(const unsigned char handle[64]) {
  std::lock_guard<std::mutex> lk(g_ipc_mu);
  std::string key((const char*)handle, 64);
  auto it = g_ipc_cache.find(key);
  if (it != g_ipc_cache.end()) {
    ++it->second.refs;
    return it->second.base;
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    fail(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
    return nullptr;
  }
  g_ipc_cache[key] = IpcMapping{p, 1};
  return p;
}

int mt_ipc_close(const unsigned char handle[64]) {
  std::lock_guard<std::mutex> lk(g_ipc_mu);
  auto it = g_ipc_cache.find(std::string((const char*)handle, 64));
  if (it == g_ipc_cache.end()) return 0;
  if (--it->second.refs <= 0) {
    cudaIpcCloseMemHandle(it->second.base);
    g_ipc_cache.erase(it);
  }
  return 0;
}

int mt_ipc_close_all(void) {
  std::lock_guard<std::mutex> lk(g_ipc_mu);
  for (auto& kv : g_ipc_cache) cudaIpcCloseMemHandle(kv.second.base);
  g_ipc_cache.clear();
  return 0;
}

// ---- collectives ------------------------------------------------------------------------------------
static int check_ready(MtComm* c) {
  if (!c || !c->d_comms) return fail("communicator is not finalized");
  return 0;
}

int mt_ring(MtComm* c, void* stream, int proto, int dtype, int op, const void* const* in, void* const* out,
            uint64_t nbytes, int root, int spatial, const int* chain, int chain_len, int nchannels) {
  if (check_ready(c)) return -1;
  // a single rank uses no FIFO, so its local-copy kernels may use as many CTAs as they like
  const int max_ch = c->nranks == 1 ? 1024 : (int)c->L.nchannels;
  if (nchannels < 1 || nchannels > max_ch) return fail("nchannels out of range");
  if (chain_len > MT_MAX_RANKS + 1) return fail("route too long");
  if (c->emulated && nchannels * c->nlocal > 148) return fail("emulated world: channels * ranks must be <= 148");
  if (c->nranks == 1 && !c->emulated && in && out && getenv("MINTCCL_NO_LOCAL_COPY") == nullptr) {
    // the only rank's contribution is the result: nothing to do in place, else one copy at HBM speed
    if (nbytes % mt::dtype_size(dtype)) return fail("byte count is not a multiple of the element size");
    if (in[0] == out[0] || nbytes == 0) return 0;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
    cudaError_t e = mt::launch_local_copy(out[0], in[0], nbytes, sms, (cudaStream_t)stream);
    if (e == cudaSuccess) {
      mthost::stat_add(mthost::ST_LOCAL_COPY, nbytes);
      return 0;
    }
    if (e != cudaErrorInvalidValue) return fail(std::string("local copy launch: ") + cudaGetErrorString(e));
    cudaGetLastError();  // pointers not co-aligned: the ring kernel copies any alignment
  }
  mt::RingArgs a;
  memset(&a, 0, sizeof(a));
  for (int lr = 0; lr < c->nlocal; ++lr) {
    a.in[lr] = in ? in[lr] : nullptr;
    a.out[lr] = out ? out[lr] : nullptr;
  }
  a.nbytes = nbytes;
  a.op = op;
  a.root = root;
  a.spatial = spatial;
  a.chain_len = chain_len;
  for (int i = 0; i < chain_len; ++i) a.chain[i] = chain[i];
  a.elem_size = mt::dtype_size(dtype);
  if (nbytes % a.elem_size) return fail("byte count is not a multiple of the element size");
  if (proto == MT_PROTO_SIMPLE && (op == mt::OP_SENDRECV || op == mt::OP_BROADCAST || op == mt::OP_REDUCE))
    a.step_bytes = mt::mt_chain_step_bytes(nbytes / (uint64_t)nchannels, c->L.fifo_slot_bytes[MT_PROTO_SIMPLE],
                                           op == mt::OP_SENDRECV ? chain_len : c->nranks);
  cudaError_t e = proto == MT_PROTO_LL128
                      ? mt::launch_ring_ll128(dtype, c->d_comms, a, nchannels, c->nlocal, (cudaStream_t)stream)
                      : mt::launch_ring_simple(dtype, c->d_comms, a, nchannels, c->nlocal, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("ring launch: ") + cudaGetErrorString(e));
  mthost::stat_add(proto == MT_PROTO_LL128 ? mthost::ST_RING_LL128 : mthost::ST_RING_SIMPLE, nbytes);
  return 0;
}

int mt_direct(MtComm* c, void* stream, int dtype, int out_dtype, int op, const void* const* in, void* const* out,
              const uint64_t* pub_in, const uint64_t* pub_out, uint64_t mc_in_off, uint64_t mc_out_off, uint64_t nbytes,
              int root, int variant, int nvls, int nctas) {
  if (check_ready(c)) return -1;
  if (nctas < 1 || nctas > 148) return fail("nctas out of range");
  if (c->emulated && nctas * c->nlocal > 148) return fail("emulated world: CTAs * ranks must be <= 148");
  if (nvls && !c->mc) return fail("NVLS requested but no multicast mapping");
  if (nvls && ((nbytes | mc_in_off | mc_out_off) & 15))
    return fail("NVLS needs heap offsets and a byte count that are multiples of 16");
  if (nbytes % mt::dtype_size(dtype)) return fail("byte count is not a multiple of the element size");
  if (root < 0 || root >= c->nranks) return fail("bad root");
  if (dtype != out_dtype) {
    if (op != mt::DOP_REDUCESCATTER && op != mt::DOP_ALLREDUCE && op != mt::DOP_REDUCE)
      return fail("only reducing collectives convert between element types");
    if (nvls || (op == mt::DOP_REDUCE && variant == 2))
      return fail("the NVLS variants do not convert between element types");
    const bool widen = (dtype == mt::DT_F16 || dtype == mt::DT_BF16) && out_dtype == mt::DT_F32;
    const bool narrow = dtype == mt::DT_F32 && (out_dtype == mt::DT_F16 || out_dtype == mt::DT_BF16);
    if (!widen && !narrow) return fail("conversions: fp16/bf16 -> fp32 and fp32 -> fp16/bf16");
  }
  if (op == mt::DOP_REDUCE && variant == 5) {
    if (dtype != out_dtype || nvls) return fail("reduce with a summing root: one element type, no NVLS");
    if (c->nranks < 3) return fail("reduce with a summing root needs at least three ranks");
    if (nbytes & 15) return fail("reduce with a summing root needs a byte count that is a multiple of 16");
    for (int lr = 0; lr < c->nlocal; ++lr)
      if ((((uintptr_t)(in ? in[lr] : nullptr)) | ((uintptr_t)(out ? out[lr] : nullptr))) & 15)
        return fail("reduce with a summing root needs 16-byte aligned buffers");
  }
  if (!c->emulated && c->nranks > 1 && (!pub_in || !pub_out)) return fail("peer views of the buffers are missing");
  mt::DirectArgs a;
  memset(&a, 0, sizeof(a));
  for (int lr = 0; lr < c->nlocal; ++lr) {
    a.in[lr] = in ? in[lr] : nullptr;
    a.out[lr] = out ? out[lr] : nullptr;
  }
  a.pub_local = c->emulated || c->nranks == 1;
  if (!a.pub_local)
    for (int p = 0; p < c->nranks; ++p) {
      a.pub_in[p] = pub_in[p];
      a.pub_out[p] = pub_out[p];
    }
  a.mc_in_off = mc_in_off;
  a.mc_out_off = mc_out_off;
  a.nbytes = nbytes;
  a.op = op;
  a.root = root;
  a.variant = variant;
  a.nvls = nvls;
  cudaError_t e = mt::launch_direct(dtype, out_dtype, c->d_comms, a, nctas, c->nlocal, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("direct launch: ") + cudaGetErrorString(e));
  mthost::stat_add(nvls ? mthost::ST_NVLS : mthost::ST_DIRECT, nbytes);
  return 0;
}

uint64_t mt_ll_capacity(MtComm* c) { return c->L.ll_bytes / MT_LL128_WARP_WIRE * MT_LL128_WARP_PAYLOAD; }

int mt_ll_allreduce(MtComm* c, void* stream, int dtype, const void* const* in, void* const* out, uint64_t nbytes) {
  if (check_ready(c)) return -1;
  if (nbytes > mt_ll_capacity(c)) return fail("message larger than the one-shot area");
  if (nbytes % mt::dtype_size(dtype)) return fail("byte count is not a multiple of the element size");
  mt::LLArgs a;
  memset(&a, 0, sizeof(a));
  for (int lr = 0; lr < c->nlocal; ++lr) {
    a.in[lr] = in[lr];
    a.out[lr] = out[lr];
  }
  a.nbytes = nbytes;
  // the grid is the same for every call so that a wire line is always served by the same CTA,
  // whose private epoch is the flag value
  cudaError_t e = mt::launch_ll_allreduce(dtype, c->d_comms, a, c->ll_grid, c->nlocal, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("ll launch: ") + cudaGetErrorString(e));
  mthost::stat_add(mthost::ST_LL_ONESHOT, nbytes);
  return 0;
}

int mt_p2p(MtComm* c, void* stream, int src_rank, int dst_rank, const void* src_ptr, void* dst_ptr, uint64_t nbytes,
           int pull, int nctas) {
  return mt_p2p_mode(c, stream, src_rank, dst_rank, src_ptr, dst_ptr, nbytes, pull, nctas, 0);
}

int mt_p2p_mode(MtComm* c, void* stream, int src_rank, int dst_rank, const void* src_ptr, void* dst_ptr, uint64_t nbytes,
                int pull, int nctas, int mode) {
  if (check_ready(c)) return -1;
  if (mode < 0 || mode > 2) return fail("bad copy mode");
  if (src_rank == dst_rank || src_rank < 0 || dst_rank < 0 || src_rank >= c->nranks || dst_rank >= c->nranks)
    return fail("bad ranks");
  if (nctas < 1 || nctas > 148) return fail("nctas out of range");
  const int copier = pull ? dst_rank : src_rank, passive = pull ? src_rank : dst_rank;
  mt::P2pArgs a;
  memset(&a, 0, sizeof(a));
  a.nbytes = nbytes;
  a.mode = mode;
  a.copier_reads_remote = pull ? 1 : 0;
  const uint64_t seq = ++c->p2p_seq[copier][passive];
  const uint64_t done = (c->p2p_done[copier][passive] += (uint64_t)nctas);
  bool any = false;
  for (int lr = 0; lr < c->nlocal; ++lr) {
    const int r = c->emulated ? lr : c->rank;
    a.src[lr] = src_ptr;
    a.dst[lr] = dst_ptr;
    a.seq[lr] = seq;
    a.done_target[lr] = done;
    if (r == copier) {
      a.role[lr] = 1;
      a.peer[lr] = passive;
      any = true;
    } else if (r == passive) {
      a.role[lr] = 2;
      a.peer[lr] = copier;
      any = true;
    }
  }
  if (!any) return 0;
  cudaError_t e = mt::launch_p2p(c->d_comms, a, nctas, c->nlocal, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("p2p launch: ") + cudaGetErrorString(e));
  mthost::stat_add(mthost::ST_P2P, nbytes);
  return 0;
}

int mt_test_wait_timeout(MtComm* c, void* stream) {
  if (check_ready(c)) return -1;
  cudaError_t e = mt::launch_wait_timeout_test(c->d_comms, c->nlocal, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("launch: ") + cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
