// Host-side state of a communicator, shared by the translation units of the runtime.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>
#include <vector>

#include "../mintccl.h"

struct MtRegService;  // host/regsrv.cpp

struct MtComm {
  int rank = 0, nranks = 1, device = 0, nlocal = 1;
  bool emulated = false;
  int heap_kind = 0;
  MtConfig cfg{};
  MtHeapLayout L{};
  uint64_t heap_bytes = 0;                 // rounded to the allocation granularity
  uint64_t timeout_ns = 0;
  // [local rank][peer] -> heap base in this process
  uint8_t* heap[MT_MAX_RANKS][MT_MAX_RANKS] = {};
  // VMM bookkeeping (real mode)
  CUmemGenericAllocationHandle local_handle = 0;
  CUmemGenericAllocationHandle peer_handle[MT_MAX_RANKS] = {};
  bool peer_mapped[MT_MAX_RANKS] = {};
  bool own_vmm = false;
  void* ipc_opened[MT_MAX_RANKS] = {};
  // multicast
  CUmemGenericAllocationHandle mc_handle = 0;
  bool mc_have_handle = false, mc_bound = false;
  uint8_t* mc = nullptr;
  int ring[MT_MAX_RANKS] = {};
  MtDevComm h_comms[MT_MAX_RANKS];
  MtDevComm* d_comms = nullptr;
  uint64_t p2p_seq[MT_MAX_RANKS][MT_MAX_RANKS] = {};
  uint64_t p2p_done[MT_MAX_RANKS][MT_MAX_RANKS] = {};
  int ll_grid = 4;
  uint64_t gemm_epoch[2] = {0, 0};         // call counters of the fused GEMM flag sets (AG, RS)
  std::vector<void*> emu_allocs;
  MtRegService* reg = nullptr;             // thread that maps the peers' ordinary allocations on request
};

namespace mthost {
// Per-family counters of successful launches through the C interface (calls and work: bytes of the message for
// collectives and copies, floating-point operations for GEMMs); read with mt_stats_get.
enum StatKind {
  ST_RING_SIMPLE = 0, ST_RING_LL128, ST_DIRECT, ST_NVLS, ST_LL_ONESHOT, ST_P2P, ST_LOCAL_COPY, ST_GEMM, ST_GEMM_MXFP8,
  ST_AG_GEMM, ST_GEMM_RS, ST_MXFP8_REDUCE, ST_COUNT
};
void stat_add(int kind, uint64_t work);
// Records an error message for mt_last_error() and returns -1.
int fail(const std::string& m);
// Looks a driver entry point up through the runtime (no link-time dependency on the driver library).
void* driver_entry(const char* name);
// TMA descriptor of a row-major [rows, K] bf16 matrix cut into box_rows x 64 tiles (128-byte swizzle).
int make_bf16_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows);
}  // namespace mthost
